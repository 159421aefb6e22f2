// Same include path as the reference; the functors live in ck/b200/element_ops.hpp.
#pragma once
#include "ck/b200/element_ops.hpp"
