// Shared device helpers: storage-dtype traits, 16-byte vector access, exact (non-contracted) fp32 arithmetic.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace opscv {

constexpr int kNumSMsFallback = 148; // B200

// ---- storage dtype <-> fp32 ------------------------------------------------------------------------------
// All interpolation arithmetic is fp32; the storage dtype is only touched on load and on the final store,
// which rounds once to nearest-even (the reference kernels cast the fp32 result to T in the same way).
template <typename T>
struct DType;
template <>
struct DType<float> {
    static constexpr bool kIsHalf = false;
    static __device__ __forceinline__ float Load(const float* p) { return __ldg(p); }
    static __device__ __forceinline__ float ToF(float v) { return v; }
    static __device__ __forceinline__ float FromF(float v) { return v; }
};
template <>
struct DType<__half> {
    static constexpr bool kIsHalf = true;
    static __device__ __forceinline__ float Load(const __half* p) { return __half2float(__ldg(p)); }
    static __device__ __forceinline__ float ToF(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half FromF(float v) { return __float2half_rn(v); }
};
template <>
struct DType<__nv_bfloat16> {
    static constexpr bool kIsHalf = false;
    // bf16 -> fp32 is exact and is just the 16 bits moved to the top half: one integer instruction, where the
    // conversion instruction would go through the (quarter-rate) conversion pipe.
    static __device__ __forceinline__ float ToF(__nv_bfloat16 v)
    {
        return __uint_as_float(static_cast<uint32_t>(__bfloat16_as_ushort(v)) << 16);
    }
    static __device__ __forceinline__ float Load(const __nv_bfloat16* p) { return ToF(__ldg(p)); }
    static __device__ __forceinline__ __nv_bfloat16 FromF(float v) { return __float2bfloat16_rn(v); }
};

// ---- 16-byte vectors of T ----------------------------------------------------------------------------------
template <typename T>
struct VecOf {
    static constexpr int kLanes = 16 / sizeof(T);
};

template <typename T, int V>
struct alignas(sizeof(T) * V) Pack {
    T v[V];
};

// Two fp32 values rounded (to nearest even, each on its own) and packed into one 32-bit register by a single
// conversion instruction; the generic path converts one at a time and then packs.
__device__ __forceinline__ uint32_t PackPair(float a, float b, const __half*)
{
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t PackPair(float a, float b, const __nv_bfloat16*)
{
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

template <typename T, int V>
__device__ __forceinline__ void StorePack(T* dst, const float (&vals)[V])
{
    if constexpr (sizeof(T) == 2 && V % 2 == 0) {
        struct alignas(sizeof(T) * V) Words {
            uint32_t w[V / 2];
        } p;
#pragma unroll
        for (int k = 0; k < V / 2; ++k) {
            p.w[k] = PackPair(vals[2 * k], vals[2 * k + 1], static_cast<const T*>(nullptr));
        }
        *reinterpret_cast<Words*>(dst) = p;
    } else {
        Pack<T, V> p;
#pragma unroll
        for (int k = 0; k < V; ++k) {
            p.v[k] = DType<T>::FromF(vals[k]);
        }
        *reinterpret_cast<Pack<T, V>*>(dst) = p;
    }
}

// One 32-byte store (sm_100 has 256-bit global stores). A thread that owns 32 contiguous bytes and writes them as two
// 16-byte stores makes every store instruction of its warp touch half of each 32-byte sector, which doubles the
// sector traffic on the SM-to-L2 path; this keeps it at one full sector per lane. dst must be 32-byte aligned.
__device__ __forceinline__ void Store32Bytes(void* dst, const uint4& lo, const uint4& hi)
{
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(lo.x), "r"(lo.y),
                 "r"(lo.z), "r"(lo.w), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
                 : "memory");
}

// The two bf16 values of a 32-bit word as fp32: the low one is the word shifted up, the high one the word masked.
// One integer instruction each; taking the halves out as 16-bit values first costs a second one (measured on the
// NHWC bilinear kernel: 6 % of its instructions).
__device__ __forceinline__ void Bf16PairToF(uint32_t w, float& lo, float& hi)
{
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
}

// fp32 values of a pack held in registers (any T)
template <typename T, int V>
__device__ __forceinline__ void UnpackToF(const Pack<T, V>& p, float (&vals)[V])
{
    if constexpr (sizeof(T) == 2 && V % 2 == 0 && !DType<T>::kIsHalf) {
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&p);
#pragma unroll
        for (int k = 0; k < V / 2; ++k) {
            Bf16PairToF(w[k], vals[2 * k], vals[2 * k + 1]);
        }
    } else {
#pragma unroll
        for (int k = 0; k < V; ++k) {
            vals[k] = DType<T>::ToF(p.v[k]);
        }
    }
}

template <typename T, int V>
__device__ __forceinline__ void LoadPack(const T* src, float (&vals)[V])
{
    const Pack<T, V> p = *reinterpret_cast<const Pack<T, V>*>(src);
    UnpackToF<T, V>(p, vals);
}

// Read-only-path version of LoadPack for 16-byte packs.
template <typename T, int V>
__device__ __forceinline__ void LoadPackLdg(const T* src, float (&vals)[V])
{
    if constexpr (sizeof(T) * V == 16) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(src));
        UnpackToF<T, V>(reinterpret_cast<const Pack<T, V>&>(raw), vals);
    } else if constexpr (sizeof(T) * V == 8) {
        const uint2 raw = __ldg(reinterpret_cast<const uint2*>(src));
        UnpackToF<T, V>(reinterpret_cast<const Pack<T, V>&>(raw), vals);
    } else {
#pragma unroll
        for (int k = 0; k < V; ++k) {
            vals[k] = DType<T>::Load(src + k);
        }
    }
}

// ---- exact fp32 arithmetic -----------------------------------------------------------------------------------
// The reference kernels are compiled without floating-point contraction; a*b+c there is two roundings. These
// wrappers keep nvcc from fusing them so that coordinates, weights and interpolated values can be compared bit
// for bit with a CPU statement of the same formulas.
__device__ __forceinline__ float Mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float Add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float Sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float Div(float a, float b) { return __fdiv_rn(a, b); }

// Packed fp32 arithmetic (sm_100: two independent IEEE round-to-nearest operations per instruction, one issue
// slot). Each half has exactly the rounding of the scalar Mul / Add / fma above, so results stay bit-identical;
// kernels whose limit is instruction issue use them on pairs of values that share an operation.
struct F2 {
    unsigned long long r; // two fp32 values in one 64-bit register: .x in the low half
};
__device__ __forceinline__ F2 MakeF2(float lo, float hi)
{
    F2 v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v.r) : "f"(lo), "f"(hi));
    return v;
}
__device__ __forceinline__ void SplitF2(F2 v, float& lo, float& hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v.r));
}
__device__ __forceinline__ F2 Mul2(F2 a, F2 b)
{
    F2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d.r) : "l"(a.r), "l"(b.r));
    return d;
}
__device__ __forceinline__ F2 Add2(F2 a, F2 b)
{
    F2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d.r) : "l"(a.r), "l"(b.r));
    return d;
}
__device__ __forceinline__ F2 Fma2(F2 a, F2 b, F2 c)
{
    F2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d.r) : "l"(a.r), "l"(b.r), "l"(c.r));
    return d;
}
// a + b on both halves when a is itself a packed product. The assembler contracts a packed multiply followed by a
// packed add into one fused multiply-add even when both carry an explicit rounding modifier (measured on sm_100a:
// 23 % of random operands came back with the fused rounding), and it sees through an fma by a literal 1.0 as
// well. A 1.0 read from constant memory is opaque to it: fma(a, 1, b) then rounds a + b once, which is the sum
// the scalar Add gives, and the product keeps its own rounding.
static __constant__ float kOpaqueOne = 1.0f;
__device__ __forceinline__ F2 AddProduct2(F2 product, F2 b)
{
    const float one = kOpaqueOne;
    return Fma2(product, MakeF2(one, one), b);
}

// row = (plane * mid + a) * inner + b. 32-bit divisions when the row count allows (`small`), which is the usual case.
__device__ __forceinline__ void SplitRow(int64_t row, int32_t inner, int32_t mid, bool small, int64_t& plane, int32_t& a,
                                         int32_t& b)
{
    if (small) {
        const uint32_t r = static_cast<uint32_t>(row);
        const uint32_t pa = r / static_cast<uint32_t>(inner);
        b = static_cast<int32_t>(r - pa * static_cast<uint32_t>(inner));
        const uint32_t p = pa / static_cast<uint32_t>(mid);
        a = static_cast<int32_t>(pa - p * static_cast<uint32_t>(mid));
        plane = p;
    } else {
        const int64_t pa = row / inner;
        b = static_cast<int32_t>(row - pa * inner);
        plane = pa / mid;
        a = static_cast<int32_t>(pa - plane * mid);
    }
}

// Launch helper: ceil-div.
__host__ __device__ __forceinline__ int64_t CeilDiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

} // namespace opscv
