#pragma once
#include "ck/b200/core.hpp"
