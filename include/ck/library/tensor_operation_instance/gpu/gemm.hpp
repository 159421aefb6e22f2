// Same include path as the reference; the factory lives in ck/b200/instance_factory.hpp.
#pragma once
#include "ck/b200/instance_factory.hpp"
