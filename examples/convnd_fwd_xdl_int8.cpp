// N-dimensional int8 forward convolution (int32 accumulation, the result keeps the low eight bits as the
// reference's static_cast does) in the style of the reference's example/09_convnd_fwd/convnd_fwd_xdl_int8.cpp:
// the fp16 driver with the reference's int8 type list (convnd_fwd_xdl_int8.cpp:23-26).
//   usage: convnd_fwd_xdl_int8 [verify init time nd [N K C <filter> <input> <strides> <dilations> <left pads> <right pads>]]
#include <cstdint>

#define CONVND_EXAMPLE_TYPES
using InDataType  = int8_t;
using WeiDataType = int8_t;
using OutDataType = int8_t;
using AccDataType = int32_t;

#include "convnd_fwd_xdl_fp16.cpp"
