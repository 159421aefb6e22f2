// Same include path as the reference; the declarations live in ck/b200/host_tensor.hpp.
#pragma once
#include "ck/b200/host_tensor.hpp"
