// Device helpers shared by the ragged-batch kernel files: activation stores (f32 rows and / or bf16 planes), small async copies,
// KV page elements (f32, or bf16 with an optional low-order plane).
#pragma once

#include "ragged.cuh"

namespace cb {
namespace {

__device__ __forceinline__ void store_act(const ActOut& o, int r, int c, float v) {
    if (o.f) o.f[(size_t)r * o.ldf + c] = v;
    if (o.hi) {
        const bf16 h = __float2bfloat16_rn(v);
        bf16* p = o.hi + (size_t)r * o.ldb + c;
        *p = h;
        if (o.lo_off) p[o.lo_off] = __float2bfloat16_rn(v - __bfloat162float(h));
    }
}

__device__ __forceinline__ void cp_async16s(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}

// KV page elements: f32, or bf16 with an optional low-order plane `lo` elements further on (x ~= hi + lo, ~16 mantissa bits)
template <typename KT> __device__ __forceinline__ float kv_load(const KT* p, long long lo);
template <> __device__ __forceinline__ float kv_load<float>(const float* p, long long) { return *p; }
template <> __device__ __forceinline__ float kv_load<bf16>(const bf16* p, long long lo) {
    const float h = __bfloat162float(*p);
    return lo ? h + __bfloat162float(p[lo]) : h;
}
template <typename KT> __device__ __forceinline__ void kv_store(KT* p, float v, long long lo);
template <> __device__ __forceinline__ void kv_store<float>(float* p, float v, long long) { *p = v; }
template <> __device__ __forceinline__ void kv_store<bf16>(bf16* p, float v, long long lo) {
    const bf16 h = __float2bfloat16_rn(v);
    *p = h;
    if (lo) p[lo] = __float2bfloat16_rn(v - __bfloat162float(h));
}

}  // namespace
}  // namespace cb
