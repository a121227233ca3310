// Shared device helpers: order-preserving logit keys, candidate records,
// Philox4x32-10, correctly rounded expf, streaming loads.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/moe_b200_sampler.h"

namespace moe {

constexpr unsigned kFullMask = 0xFFFFFFFFu;

// ---- order-preserving keys ----------------------------------------------------
// The reference ranks by `values[left] > values[right]`, index ascending on
// `==` (src/engine/session.cpp:26-36).  -0.0 == +0.0 there, so the sign of a
// zero is dropped before the bits are made monotone.  NaN never gets a key:
// callers filter it with float compares first.
__device__ __forceinline__ uint32_t ordered_key(float value)
{
    const uint32_t bits = __float_as_uint(value + 0.0f);
    return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

__device__ __forceinline__ float key_to_float(uint32_t key)
{
    const uint32_t bits = (key & 0x80000000u) ? (key & 0x7FFFFFFFu) : ~key;
    return __uint_as_float(bits);
}

constexpr uint32_t kKeyNegInf = 0x007FFFFFu; // ordered_key(-inf)
constexpr uint32_t kKeyPosInf = 0xFF800000u; // ordered_key(+inf)

// A candidate record: larger record = earlier in the reference rank order
// (higher logit first, then lower token id).  0 is never a valid record
// because kKeyNegInf > 0.
__device__ __forceinline__ uint64_t make_record(uint32_t key, uint32_t index)
{
    return (static_cast<uint64_t>(key) << 32) | static_cast<uint64_t>(0xFFFFFFFFu - index);
}
__device__ __forceinline__ uint32_t record_key(uint64_t record)
{
    return static_cast<uint32_t>(record >> 32);
}
__device__ __forceinline__ uint32_t record_index(uint64_t record)
{
    return 0xFFFFFFFFu - static_cast<uint32_t>(record);
}

// ---- Philox4x32-10 (Salmon et al., SC'11) -------------------------------------
__host__ __device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1,
                                                        uint32_t (&out)[4])
{
#pragma unroll
    for (int round = 0; round < 10; ++round)
    {
        const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c0;
        const uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c2;
        const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c1 ^ k0;
        const uint32_t n1 = static_cast<uint32_t>(p1);
        const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c3 ^ k1;
        const uint32_t n3 = static_cast<uint32_t>(p0);
        c0 = n0;
        c1 = n1;
        c2 = n2;
        c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    out[0] = c0;
    out[1] = c1;
    out[2] = c2;
    out[3] = c3;
}

// key = seed, counter = (row_id, step); uniform = top 24 bits of word 0.
__host__ __device__ __forceinline__ float philox_uniform(uint64_t seed, uint64_t row_id, uint64_t step)
{
    uint32_t words[4];
    philox4x32_10(static_cast<uint32_t>(row_id), static_cast<uint32_t>(row_id >> 32), static_cast<uint32_t>(step),
                  static_cast<uint32_t>(step >> 32), static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32), words);
    return static_cast<float>(words[0] >> 8) * 5.9604644775390625e-08f; // 2^-24
}

// ---- arithmetic that must round like the host ----------------------------------
// expf rounded once from a double-precision exp: the correctly rounded float
// result (up to double rounding, ~1e-9 of arguments).  The host libm's expf is
// itself correctly rounded for all but ~6e-4 of arguments, where it is one ulp
// off; the fast device expf (2 ulp) would be much further away.
__device__ __forceinline__ float exact_expf(float x)
{
    return __double2float_rn(exp(static_cast<double>(x)));
}
__device__ __forceinline__ float exact_log1pf(float x)
{
    return __double2float_rn(log1p(static_cast<double>(x)));
}

// `logit / temperature - peak` exactly as session.cpp:98 evaluates it: one
// rounded division, one rounded subtraction, no contraction.
__device__ __forceinline__ float scaled_offset(float logit, float temperature, float peak)
{
    return __fsub_rn(__fdiv_rn(logit, temperature), peak);
}

// ---- streaming 128-bit loads ----------------------------------------------------
// Logits are read exactly once: read-only path, no L1 allocation.
__device__ __forceinline__ uint4 load_stream_16(const void* pointer)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(pointer));
    return v;
}

// ---- shared-memory accesses with the state space spelled out -------------------
// A pointer into dynamic shared memory that has travelled through a struct or a
// function argument is a generic pointer to the compiler, and generic loads go
// down the global-memory path (long-scoreboard latency) before they reach
// shared memory.  The hot loops therefore address shared memory by its 32-bit
// window address.
__device__ __forceinline__ uint32_t shared_address(const void* pointer)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}
__device__ __forceinline__ uint4 load_shared_16(uint32_t address)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(address));
    return v;
}
__device__ __forceinline__ void store_shared_16(uint32_t address, const uint4& v)
{
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(address), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ ulonglong2 load_shared_2x64(uint32_t address)
{
    ulonglong2 v;
    asm volatile("ld.shared.v2.u64 {%0,%1}, [%2];" : "=l"(v.x), "=l"(v.y) : "r"(address));
    return v;
}
__device__ __forceinline__ uint64_t load_shared_64(uint32_t address)
{
    unsigned long long v;
    asm volatile("ld.shared.u64 %0, [%1];" : "=l"(v) : "r"(address));
    return v;
}
__device__ __forceinline__ void store_shared_64(uint32_t address, uint64_t v)
{
    asm volatile("st.shared.u64 [%0], %1;" ::"r"(address), "l"(static_cast<unsigned long long>(v)) : "memory");
}
__device__ __forceinline__ uint32_t load_shared_32(uint32_t address)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(address));
    return v;
}
__device__ __forceinline__ uint32_t load_shared_32_volatile(uint32_t address)
{
    uint32_t v;
    asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(v) : "r"(address) : "memory");
    return v;
}
__device__ __forceinline__ void store_shared_32(uint32_t address, uint32_t v)
{
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(address), "r"(v) : "memory");
}
__device__ __forceinline__ float load_shared_f32(uint32_t address)
{
    return __uint_as_float(load_shared_32(address));
}
__device__ __forceinline__ uint32_t atomic_add_shared(uint32_t address, uint32_t value)
{
    uint32_t old;
    asm volatile("atom.shared.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(address), "r"(value) : "memory");
    return old;
}
__device__ __forceinline__ void atomic_max_shared(uint32_t address, uint32_t value)
{
    asm volatile("red.shared.max.u32 [%0], %1;" ::"r"(address), "r"(value) : "memory");
}

template<typename T>
struct LogitTraits;

template<>
struct LogitTraits<float>
{
    static constexpr int kPerVector = 4;
    __device__ static __forceinline__ float widen(const float* pointer, size_t index)
    {
        return pointer[index];
    }
};

template<>
struct LogitTraits<__nv_bfloat16>
{
    static constexpr int kPerVector = 8;
    __device__ static __forceinline__ float widen(const __nv_bfloat16* pointer, size_t index)
    {
        return __uint_as_float(static_cast<uint32_t>(reinterpret_cast<const uint16_t*>(pointer)[index]) << 16);
    }
};

// ---- warp / block reductions ------------------------------------------------------
__device__ __forceinline__ uint32_t warp_max_u32(uint32_t v)
{
    return __reduce_max_sync(kFullMask, v);
}

__device__ __forceinline__ uint64_t warp_or_u64(uint64_t v)
{
    const uint32_t lo = __reduce_or_sync(kFullMask, static_cast<uint32_t>(v));
    const uint32_t hi = __reduce_or_sync(kFullMask, static_cast<uint32_t>(v >> 32));
    return (static_cast<uint64_t>(hi) << 32) | lo;
}
__device__ __forceinline__ uint64_t warp_and_u64(uint64_t v)
{
    const uint32_t lo = __reduce_and_sync(kFullMask, static_cast<uint32_t>(v));
    const uint32_t hi = __reduce_and_sync(kFullMask, static_cast<uint32_t>(v >> 32));
    return (static_cast<uint64_t>(hi) << 32) | lo;
}

// Per-row parameter validation in the order of validate_sampling_options
// (src/engine/session.cpp:65-74).
__host__ __device__ __forceinline__ int validate_row(const moe_row_params& p)
{
    const bool t_ok = (p.temperature == p.temperature) && (p.temperature - p.temperature == 0.0f) && p.temperature >= 0.0f;
    if (!t_ok)
        return MOE_ROW_BAD_TEMPERATURE;
    const bool p_ok = (p.top_p - p.top_p == 0.0f) && p.top_p > 0.0f && p.top_p <= 1.0f;
    if (!p_ok)
        return MOE_ROW_BAD_TOP_P;
    const bool m_ok = (p.min_p - p.min_p == 0.0f) && p.min_p >= 0.0f && p.min_p <= 1.0f;
    if (!m_ok)
        return MOE_ROW_BAD_MIN_P;
    return MOE_ROW_OK;
}

} // namespace moe
