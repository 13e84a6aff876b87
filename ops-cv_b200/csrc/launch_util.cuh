// Launch-configuration helpers shared by the .cu files: dtype dispatch, vector-width choice, grid sizing.
#pragma once

#include <initializer_list>
#include <type_traits>

#include "common.cuh"
#include "kernels.h"

namespace opscv {

// Number of SMs of the current device (cached per thread; 148 on B200).
int NumSMs();

// Grid for a grid-stride kernel over `items` work items with `threads` threads per block: enough blocks to cover
// the items once, capped at `wavesCap` resident-block multiples of the SM count so the grid is a multiple of the
// SM count whenever the problem is large.
inline unsigned GridFor(int64_t items, int threads, int blocksPerSm = 8)
{
    const int64_t need = CeilDiv(items, threads);
    const int64_t cap = static_cast<int64_t>(NumSMs()) * blocksPerSm;
    int64_t g = need < cap ? need : cap;
    if (g < 1) {
        g = 1;
    }
    return static_cast<unsigned>(g);
}

// Block shape (column threads, row threads) of the plane-tile kernels: one thread per column group, and as many
// row threads as keep about `rowsPerThread` rows of the tile for each of them (long walks reuse more).
inline dim3 TileBlock(int32_t groups, int32_t rows, int32_t rowsPerThread = 16)
{
    int32_t ct = groups < 256 ? groups : 256;
    ct = ct < 1 ? 1 : ct;
    int32_t rt = 256 / ct;
    const int32_t wantRt = (rows + rowsPerThread - 1) / rowsPerThread;
    rt = rt < wantRt ? rt : wantRt;
    rt = rt < 1 ? 1 : rt;
    return dim3(static_cast<unsigned>(ct), static_cast<unsigned>(rt), 1);
}

// Launch shape of the row kernels of the 3-D resamplers: a block is (column threads) x (row threads) with 256 threads
// in all, the column side just wide enough for the `colItems` threads a row needs (a power of two), so that narrow
// rows keep all lanes busy; grid.y walks the rows and is capped so that the grid stays near 16 blocks per SM.
struct RowLaunch {
    dim3 grid, block;
};
inline RowLaunch RowTiling(int64_t rows, int64_t colItems, int threads = 256)
{
    int ct = 1;
    while (ct < colItems && ct < threads) {
        ct <<= 1;
    }
    const int rt = threads / ct;
    const int64_t colBlocks = CeilDiv(colItems, static_cast<int64_t>(ct));
    const int64_t rowBlocks = CeilDiv(rows < 1 ? 1 : rows, static_cast<int64_t>(rt));
    int64_t cap = static_cast<int64_t>(NumSMs()) * 16 / (colBlocks < 1 ? 1 : colBlocks);
    cap = cap < 1 ? 1 : cap;
    int64_t gy = rowBlocks < cap ? rowBlocks : cap;
    gy = gy < 65535 ? gy : 65535;
    RowLaunch r;
    r.grid = dim3(static_cast<unsigned>(colBlocks), static_cast<unsigned>(gy), 1);
    r.block = dim3(static_cast<unsigned>(ct), static_cast<unsigned>(rt), 1);
    return r;
}

inline bool Aligned(const void* p, size_t bytes) { return (reinterpret_cast<uintptr_t>(p) % bytes) == 0; }

// Largest vector width (in elements, power of two, at most 16 bytes) such that `inner` is a multiple of it and
// every pointer is aligned to the vector size.
inline int PickVec(int elemSize, int64_t inner, std::initializer_list<const void*> ptrs)
{
    for (int v = 16 / elemSize; v > 1; v >>= 1) {
        if (inner % v != 0) {
            continue;
        }
        bool ok = true;
        for (const void* p : ptrs) {
            ok = ok && Aligned(p, static_cast<size_t>(v) * elemSize);
        }
        if (ok) {
            return v;
        }
    }
    return 1;
}

#define OPSCV_DISPATCH_DT(dt, T, ...)                 \
    switch (dt) {                                     \
        case Dt::F32: {                               \
            using T = float;                          \
            __VA_ARGS__;                              \
            break;                                    \
        }                                             \
        case Dt::F16: {                               \
            using T = __half;                         \
            __VA_ARGS__;                              \
            break;                                    \
        }                                             \
        case Dt::BF16: {                              \
            using T = __nv_bfloat16;                  \
            __VA_ARGS__;                              \
            break;                                    \
        }                                             \
    }

// Dispatch a vector width chosen at run time onto a compile-time constant. The body runs inside a generic lambda
// so that `if constexpr (V * sizeof(T) <= 16)` really discards the over-wide instantiations.
#define OPSCV_DISPATCH_VEC(v, V, ...)                                  \
    {                                                                  \
        auto opscvBody_ = [&](auto opscvTag_) {                        \
            constexpr int V = decltype(opscvTag_)::value;              \
            __VA_ARGS__;                                               \
        };                                                             \
        switch (v) {                                                   \
            case 8: opscvBody_(std::integral_constant<int, 8>{}); break; \
            case 4: opscvBody_(std::integral_constant<int, 4>{}); break; \
            case 2: opscvBody_(std::integral_constant<int, 2>{}); break; \
            default: opscvBody_(std::integral_constant<int, 1>{}); break; \
        }                                                              \
    }

} // namespace opscv
