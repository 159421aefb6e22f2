// device_utility/device_prop.hpp:12-52
#pragma once
#include <string>
#include "ckb200.h"
namespace ck {
inline std::string get_device_name()
{
    char name[256] = {0};
    ckb_device_info(name, sizeof(name), nullptr, nullptr, nullptr);
    return name;
}
} // namespace ck
