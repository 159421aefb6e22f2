// Same include path as the reference; the declarations live in ck/b200/device_ops.hpp.
#pragma once
#include "ck/b200/device_ops.hpp"
