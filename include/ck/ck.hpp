// Drop-in for the reference's include/ck/ck.hpp (basic types and configuration).
#pragma once
#include "ck/b200/core.hpp"

#define CK_TIME_KERNEL 1 // include/ck/ck.hpp:11
