// Same include path as the reference; the operators live in ck/b200/reference_ops.hpp.
#pragma once
#include "ck/b200/reference_ops.hpp"
