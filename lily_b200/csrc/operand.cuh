// A kernel input that is [rows, cols] in bfloat16 or float32, or the float32 partial sums of a split-k product
// ([splits][rows, cols], `stride` elements apart), which are added up in order while they are read.
#pragma once

#include "common.cuh"

namespace lily {

struct Operand {
    const void* p;
    int bf16;
    int splits;
    size_t stride;
    __device__ __forceinline__ float operator()(size_t i) const {
        if (bf16) return __bfloat162float(((const __nv_bfloat16*)p)[i]);
        const float* f = (const float*)p;
        float v = f[i];
        for (int s = 1; s < splits; ++s) v += f[i + (size_t)s * stride];
        return v;
    }
    // four consecutive entries from a multiple of four (16-byte aligned base, stride a multiple of four)
    __device__ __forceinline__ float4 four(size_t i) const {
        if (bf16) {
            const uint2 raw = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)p + i);
            const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
            const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
            return make_float4(lo.x, lo.y, hi.x, hi.y);
        }
        const float* f = (const float*)p;
        float4 v = *reinterpret_cast<const float4*>(f + i);
        for (int s = 1; s < splits; ++s) {
            const float4 t = *reinterpret_cast<const float4*>(f + i + (size_t)s * stride);
            v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
        }
        return v;
    }
    bool vector_ok() const { return p == nullptr || (((uintptr_t)p & 15) == 0 && stride % 4 == 0); }
};

}  // namespace lily
