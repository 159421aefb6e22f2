// Same include path as the reference; the declarations live in ck/b200/host_utility.hpp.
#pragma once
#include "ck/b200/host_utility.hpp"
