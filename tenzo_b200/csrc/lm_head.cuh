// Shared between the two LM-head kernels (lm_head.cu, lm_head_umma.cu): the argmax candidate record
// and its ordering.
#pragma once

namespace tz {

struct LmBest { float val; int idx; };

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
    // greedy argmax keeps the first maximum (TenzoEngine.cpp:1749 of the reference, strict '>'):
    // larger value, or same value at a lower index
    return v > bv || (v == bv && i < bi);
}

constexpr int kLmuMaxTiles = 2048;   // 128-row vocabulary tiles the tensor-core path's scratch is sized for (vocab <= 262144)

}  // namespace tz
