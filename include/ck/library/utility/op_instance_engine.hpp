// Same include path as the reference; the engine lives in ck/b200/op_instance_engine.hpp.
#pragma once
#include "ck/b200/op_instance_engine.hpp"
