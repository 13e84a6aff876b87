// Shared-memory staging of the rows of one NCHW plane that an output tile reads.
//
// The gathers of the resamplers have strong locality (an output row reads one or two input rows, neighbouring
// outputs read neighbouring inputs) but, issued straight to global memory, every scalar gather makes L1 look up
// the same 32-byte sectors again and again: the first version of these kernels was bound by L1 sector
// throughput at ~25% of HBM bandwidth. Staging turns the global reads into one fully coalesced 16-byte-per-thread
// copy of a contiguous span (each sector requested once) and moves the gathers to shared memory.
#pragma once

#include "common.cuh"

namespace opscv {

// Copies `count` consecutive elements starting at `src` (global) into shared memory and returns the shared
// pointer p with p[k] == src[k]. `raw` must be 16-byte aligned and hold count * sizeof(T) + 16 bytes: the copy is
// shifted so that shared and global addresses are congruent modulo 16, which lets the body move as uint4.
// All threads of the (1-D or 2-D) block must call it; the caller synchronises afterwards.
template <typename T>
__device__ __forceinline__ T* StageSpan(const T* __restrict__ src, int64_t count, unsigned char* raw)
{
    constexpr int kPer = 16 / sizeof(T);
    const int mis = static_cast<int>((reinterpret_cast<uintptr_t>(src) & 15) / sizeof(T));
    T* dst = reinterpret_cast<T*>(raw) + mis;
    int64_t head = (kPer - mis) % kPer;
    if (head > count) {
        head = count;
    }
    const int64_t body = (count - head) / kPer;
    const int64_t tailStart = head + body * kPer;
    const int32_t tid = threadIdx.y * blockDim.x + threadIdx.x, nthreads = blockDim.x * blockDim.y;
    for (int64_t i = tid; i < head; i += nthreads) {
        dst[i] = __ldg(src + i);
    }
    const uint4* s4 = reinterpret_cast<const uint4*>(src + head);
    uint4* d4 = reinterpret_cast<uint4*>(dst + head);
    for (int64_t i = tid; i < body; i += nthreads) {
        d4[i] = __ldg(s4 + i);
    }
    for (int64_t i = tailStart + tid; i < count; i += nthreads) {
        dst[i] = __ldg(src + i);
    }
    return dst;
}

inline size_t StageBytes(int64_t count, int elemSize) { return static_cast<size_t>(count) * elemSize + 16; }

// Rows of a tile: how many output rows a block takes so that the input rows it needs fit in `budget` bytes.
// needRows(t) must be a non-decreasing upper bound of the input rows needed by t consecutive output rows.
template <typename F>
inline int32_t PickTileRows(int32_t outRows, int64_t rowBytes, int64_t budget, F needRows)
{
    int32_t lo = 1, hi = outRows;
    if (static_cast<int64_t>(needRows(hi)) * rowBytes <= budget) {
        return hi;
    }
    while (lo < hi) { // largest t with needRows(t) * rowBytes <= budget (0 if none)
        const int32_t mid = lo + (hi - lo + 1) / 2;
        if (static_cast<int64_t>(needRows(mid)) * rowBytes <= budget) {
            lo = mid;
        } else {
            hi = mid - 1;
        }
    }
    return static_cast<int64_t>(needRows(lo)) * rowBytes <= budget ? lo : 0;
}

} // namespace opscv
