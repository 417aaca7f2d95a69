// Host-side helpers shared by the attention translation units (implemented in kvq_decode.cu).
#pragma once
#include <cuda.h>

#include <cstdint>

namespace kvq {

// Number of SMs of the current device (cached); also makes sure the driver's tensor-map encoder is resolved.
int shared_device_sms(int* sms);

// Tensor map over an int8 cache view [nb, bs, H, D] with boxes of 16 slots x box_heads heads x D channels
// (128-byte swizzle for D = 128, 64-byte for D = 64). The three outer dims are ordered by stride; pos[0..2]
// receive the coordinate slot (1..3) that holds the (slot-in-block, head, block) index. Maps are cached.
int shared_cache_tensor_map(const void* ptr, int64_t nb, int bs, int H, int D, int64_t sb, int64_t sn, int64_t sh,
                            int box_heads, CUtensorMap* map, int* pos);

}  // namespace kvq
