// UpsampleBilinear2d forward and backward.
//
// The reference formula  (1-dy)*((1-dx)*TL + dx*TR) + dy*((1-dx)*BL + dx*BR)  is a vertical blend of two
// horizontally interpolated input rows. All NCHW forward kernels use that: a thread owns a group of output columns,
// walks down a run of output rows, keeps the horizontal interpolation of the current top and bottom input rows in
// registers and touches memory only when the walk reaches a new input row. The operation order is the
// reference's, so results are bit-identical to it.
//
// Kernel schedules (chosen on the host from exact copies of the index tables, see MakeBilinearFwdPlan /
// MakeBilinearBwdPlan):
//   * NCHW, output width = 2 x input width (FPN-style up-sampling): input-major. A thread loads one vector of four
//     input columns (plus one neighbour on each side) per input row and produces the eight output columns they
//     feed; loads and stores are coalesced vectors and every input element is fetched once per row walk.
//     The backward is the transpose: a thread loads eight grads columns (plus neighbours) per grads row, reduces
//     them to four grad_input columns and adds the row, with its two vertical weights, to the (at most two)
//     grad_input rows it touches.
//   * NCHW, any other scale: the same walks over shared memory. A block copies the rows its band reads into shared
//     memory (coalesced 16-byte loads, tile_stage.cuh); horizontal taps are shared-memory reads.
//   * NCHW rows too long to stage, user scales that overshoot the input, unaligned tensors: direct kernels.
//   * NHWC: a thread owns 16 bytes of channels of one pixel; taps are 16-byte global loads.
// Backward results are reproducible in every schedule (fixed summation order, no atomics). The direct and NHWC
// backward kernels add the reference scatter kernel's products in its serial order and equal it bit for bit; the
// row-walk kernels reduce rows first (separable, fused multiply-add) and agree to fp32 rounding.
// The atomic scatter (the reference's non-deterministic schedule) is kept selectable; it is slower here.
//
// Reference arithmetic: image/resize_bilinear_v2/op_kernel/arch35/resize_bilinear_v2_simt_nchw.h:84-146,
// _simt_nhwc.h:88-151; image/resize_bilinear_v2_grad/op_kernel/arch35/resize_bilinear_v2_grad_simt.h:107-152.
#include <algorithm>
#include <cstring>
#include <type_traits>

#include "host_tables.h"
#include "launch_util.cuh"
#include "cp_async.cuh"
#include "lerp_entry.cuh"
#include "tile_stage.cuh"

namespace opscv {
namespace {

constexpr int kThreads = 256;
constexpr int64_t kStageBudget = 40 * 1024; // staged bytes per block: 5 blocks resident per SM

// ---- forward, NCHW ----------------------------------------------------------------------------------------
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    BilinearFwdNCHWKernel(const T* __restrict__ x, T* __restrict__ y, int32_t hin, int32_t win, int32_t hout,
                          int32_t wout, LerpAxis th, LerpAxis tw, int32_t rowsPerThread, int32_t rowChunks,
                          int64_t totalThreads)
{
    const int32_t groups = wout / V;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; tid < totalThreads; tid += stride) {
        const int64_t pc = tid / groups;
        const int32_t g = static_cast<int32_t>(tid - pc * groups);
        const int64_t p = pc / rowChunks;
        const int32_t chunk = static_cast<int32_t>(pc - p * rowChunks);
        int32_t wl[V], wh[V];
        float dx[V], dx1[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            wl[k] = __ldg(tw.lo + g * V + k);
            wh[k] = __ldg(tw.hi + g * V + k);
            dx[k] = __ldg(tw.delta + g * V + k);
            dx1[k] = Sub(1.0f, dx[k]);
        }
        const T* xp = x + p * hin * static_cast<int64_t>(win);
        T* yp = y + p * hout * static_cast<int64_t>(wout) + static_cast<int64_t>(g) * V;
        float top[V], bot[V];
        int32_t curTop = -1, curBot = -1;
        const int32_t h0 = chunk * rowsPerThread;
        const int32_t h1 = min(hout, h0 + rowsPerThread);
        for (int32_t h = h0; h < h1; ++h) {
            const int32_t lo = __ldg(th.lo + h), hi = __ldg(th.hi + h);
            const float dy = __ldg(th.delta + h);
            if (lo != curTop) {
                if (lo == curBot) {
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        top[k] = bot[k];
                    }
                } else {
                    const T* xr = xp + static_cast<int64_t>(lo) * win;
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        top[k] = Add(Mul(dx1[k], DType<T>::Load(xr + wl[k])), Mul(dx[k], DType<T>::Load(xr + wh[k])));
                    }
                }
                curTop = lo;
            }
            if (hi != curBot) {
                if (hi == curTop) {
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        bot[k] = top[k];
                    }
                } else {
                    const T* xr = xp + static_cast<int64_t>(hi) * win;
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        bot[k] = Add(Mul(dx1[k], DType<T>::Load(xr + wl[k])), Mul(dx[k], DType<T>::Load(xr + wh[k])));
                    }
                }
                curBot = hi;
            }
            const float dy1 = Sub(1.0f, dy);
            float out[V];
#pragma unroll
            for (int k = 0; k < V; ++k) {
                out[k] = Add(Mul(dy1, top[k]), Mul(dy, bot[k]));
            }
            StorePack<T, V>(yp + static_cast<int64_t>(h) * wout, out);
        }
    }
}

// Vertical blend shared by the forward walks: given the horizontal interpolations of the top and bottom rows.
template <typename T, int V>
__device__ __forceinline__ void BlendStore(T* dst, const float (&top)[V], const float (&bot)[V], float dy,
                                           bool wide = false)
{
    const float dy1 = Sub(1.0f, dy);
    // out = dy1 * top + dy * bot with the reference's three roundings, two values per instruction: packed multiplies
    // and an exact packed add of the products (AddProduct2), which halves the issue slots of the blend.
    const F2 wTop = MakeF2(dy1, dy1), wBot = MakeF2(dy, dy);
    auto blend = [&](int k, float& a, float& b) { // outputs k and k + 1
        const F2 r = AddProduct2(Mul2(wBot, MakeF2(bot[k], bot[k + 1])), Mul2(wTop, MakeF2(top[k], top[k + 1])));
        SplitF2(r, a, b);
    };
    if constexpr (V * sizeof(T) == 32) {
        if (wide) { // dst is 32-byte aligned: one full-sector store per lane
            Pack<T, V / 2> half[2];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                float out[V / 2];
#pragma unroll
                for (int k = 0; k < V / 2; k += 2) {
                    blend(q * (V / 2) + k, out[k], out[k + 1]);
                }
                StorePack<T, V / 2>(half[q].v, out);
            }
            Store32Bytes(dst, reinterpret_cast<const uint4&>(half[0]), reinterpret_cast<const uint4&>(half[1]));
            return;
        }
    }
    constexpr int kPer = (V * sizeof(T) > 16) ? 16 / sizeof(T) : V; // at most 16 bytes per store
#pragma unroll
    for (int q = 0; q < V / kPer; ++q) {
        float out[kPer];
        if constexpr (kPer % 2 == 0) {
#pragma unroll
            for (int k = 0; k < kPer; k += 2) {
                blend(q * kPer + k, out[k], out[k + 1]);
            }
        } else {
#pragma unroll
            for (int k = 0; k < kPer; ++k) {
                out[k] = Add(Mul(dy1, top[q * kPer + k]), Mul(dy, bot[q * kPer + k]));
            }
        }
        StorePack<T, kPer>(dst + q * kPer, out);
    }
}

// ---- forward, NCHW, shared-memory staged ---------------------------------------------------------------------
// grid = (plane groups, tiles per plane), block = (column threads, planes). A tile is `tileRows` output rows; its
// input rows [lo[h0], hi[h1-1]] are staged for every plane of the block (the host sized the tile so that they fit).
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    BilinearFwdTileKernel(const T* __restrict__ x, T* __restrict__ y, int64_t planes, int32_t hin, int32_t win,
                          int32_t hout, int32_t wout, LerpAxis th, LerpAxis tw, int32_t tileRows, int32_t stageStride)
{
    extern __shared__ __align__(16) unsigned char smemRaw[];
    // block = (column threads, planes): the bands of blockDim.y planes are staged, `stageStride` bytes apart
    const int64_t pBase = static_cast<int64_t>(blockIdx.x) * blockDim.y;
    const int32_t np = static_cast<int32_t>(min(static_cast<int64_t>(blockDim.y), planes - pBase));
    const int32_t ha = blockIdx.y * tileRows, hb = min(hout, ha + tileRows);
    const int32_t r0 = __ldg(th.lo + ha), r1 = __ldg(th.hi + hb - 1) + 1;
    const int64_t planeElems = hin * static_cast<int64_t>(win);
    const T* src = nullptr;
    for (int32_t pl = 0; pl < np; ++pl) {
        const T* staged = StageSpan<T>(x + (pBase + pl) * planeElems + static_cast<int64_t>(r0) * win,
                                       static_cast<int64_t>(r1 - r0) * win, smemRaw + pl * stageStride);
        if (pl == static_cast<int32_t>(threadIdx.y)) {
            src = staged;
        }
    }
    __syncthreads();
    if (static_cast<int32_t>(threadIdx.y) >= np) {
        return;
    }
    const int64_t p = pBase + threadIdx.y;
    const int32_t groups = wout / V;
    const int32_t colThreads = blockDim.x, cg0 = threadIdx.x;
    T* yp = y + p * hout * static_cast<int64_t>(wout);
    for (int32_t g = cg0; g < groups; g += colThreads) {
        int32_t wl[V], wh[V];
        float dx[V], dx1[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            wl[k] = __ldg(tw.lo + g * V + k);
            wh[k] = __ldg(tw.hi + g * V + k);
            dx[k] = __ldg(tw.delta + g * V + k);
            dx1[k] = Sub(1.0f, dx[k]);
        }
        float top[V], bot[V];
        int32_t curTop = -1, curBot = -1;
        T* dst = yp + static_cast<int64_t>(ha) * wout + g * V;
        for (int32_t h = ha; h < hb; ++h) {
            const int32_t lo = __ldg(th.lo + h), hi = __ldg(th.hi + h);
            if (lo != curTop) {
                if (lo == curBot) {
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        top[k] = bot[k];
                    }
                } else {
                    const T* xr = src + (lo - r0) * win;
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        top[k] = Add(Mul(dx1[k], DType<T>::ToF(xr[wl[k]])), Mul(dx[k], DType<T>::ToF(xr[wh[k]])));
                    }
                }
                curTop = lo;
            }
            if (hi != curBot) {
                if (hi == curTop) {
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        bot[k] = top[k];
                    }
                } else {
                    const T* xr = src + (hi - r0) * win;
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        bot[k] = Add(Mul(dx1[k], DType<T>::ToF(xr[wl[k]])), Mul(dx[k], DType<T>::ToF(xr[wh[k]])));
                    }
                }
                curBot = hi;
            }
            BlendStore<T, V>(dst, top, bot, __ldg(th.delta + h));
            dst += wout;
        }
    }
}

// ---- per-thread asynchronous row queues ------------------------------------------------------------------------
// The row walks below are serial chains per thread, so what bounds them is the number of bytes a thread has in
// flight. cp.async copies a thread's own piece of the next rows into a private shared-memory queue (one commit
// group per row, cp.async.wait_group to consume in order), which holds several times what registers could.
// ---- forward, NCHW, output width = 2 x input width, input-major ---------------------------------------------------
// The host has verified the column pattern lo[w] = max((w-1)>>1, 0), hi[w] = w ? min((w+1)>>1, win-1) : 0, so the
// 2*VI outputs of input columns c0..c0+VI-1 read columns c0-1..c0+VI (clamped). Weights still come from the table.
// grid = (plane groups, tiles per plane), block = (column threads, planes); rows are table-driven (any vertical
// scale).
constexpr int kFwdQueueDepth = 4; // NHWC column walker
constexpr int kW2QueueDepth = 4;  // 2x-width row walker (8 measured the same)

// QUEUE (needs VI * sizeof(T) == 16): the input rows stream through a per-thread cp.async queue.
// PERIODIC: the column weights are the three scalars (dxFirst for output column 0, dxEven, dxOdd) instead of tw.delta.
// Seven warps per block: three resident blocks then leave 96 registers per thread, which the two row buffers of the
// 16-column variant need (at 256 threads and 80 registers the walk spilled and recomputed its weights).
constexpr int kW2Threads = 128;

// FUSE (with PERIODIC, 16-bit T): the host has checked that every column weight times any value of T is exact in
// fp32, so the horizontal interpolation may use one fused multiply-add: same bits, one instruction fewer.
// PITCH: the output is a view addressed through outPitch (N, C, H pitches); otherwise the dense expressions are kept
// as they were, so that the dense kernel's code does not change.
// X2ROWS (with PERIODIC): the host has checked that the row table is the 2x pattern (row 0 from input row 0 alone, rows
// 2i + 1 and 2i + 2 from input rows i and i + 1, the last row from the last input row alone); a tile's rows are then
// walked in a straight line, one new input row per two output rows, the two row buffers trading places in a loop
// body written twice, instead of comparing every row's entry with the rows held. Same loads, same blends.
template <typename T, int VI, bool QUEUE, bool PERIODIC, bool FUSE = false, bool PITCH = false, bool X2ROWS = false>
__global__ void __launch_bounds__(kW2Threads, 5)
    BilinearFwdW2Kernel(const T* __restrict__ x, T* __restrict__ y, int64_t planes, int32_t hin, int32_t win,
                        int32_t hout, LerpAxis th, LerpAxis tw, int32_t tileRows, int32_t wideStores, float dxFirst,
                        float dxEven, float dxOdd, AxisGeom geomH, int32_t halfPixel, ViewStrides outPitch,
                        ViewStrides inPitch)
{
    constexpr int VO = 2 * VI;
    constexpr int HE = 4 / sizeof(T); // elements in a 4-byte neighbour word
    extern __shared__ __align__(16) unsigned char fwdQueue[];
    const int32_t tid = threadIdx.y * blockDim.x + threadIdx.x, nthreads = blockDim.x * blockDim.y;
    // PERIODIC: [tileRows] row entries {lo, hi, delta} of the tile, evaluated by the block itself (this variant reads
    // no table, so none has to be built before it); then
    // [depth][nthreads] 16-byte vectors, then the left and right neighbour words
    float4* rowT = reinterpret_cast<float4*>(fwdQueue);
    uint4* qMid = reinterpret_cast<uint4*>(fwdQueue) + (PERIODIC ? tileRows : 0);
    uint32_t* qLeft = reinterpret_cast<uint32_t*>(qMid + static_cast<size_t>(kW2QueueDepth) * nthreads);
    uint32_t* qRight = qLeft + static_cast<size_t>(kW2QueueDepth) * nthreads;
    const int32_t wout = 2 * win;
    // block = (column threads, planes): every thread of a block walks the same rows, so the row logic is uniform.
    // The output rows of all plane groups form one sequence (group-major); the blocks cut it into gridDim.x equal
    // runs, so that one wave of resident blocks finishes together whatever the number of planes. A run is walked as
    // tiles: its pieces of consecutive plane groups, none taller than tileRows.
    const int64_t planeGroups = (planes + blockDim.y - 1) / blockDim.y;
    const int64_t totalRows = planeGroups * hout;
    const int64_t share = totalRows / gridDim.x, rest = totalRows - share * gridDim.x; // the first `rest` runs get one more
    int64_t pos = share * blockIdx.x + min(static_cast<int64_t>(blockIdx.x), rest);
    const int64_t end = pos + share + (blockIdx.x < rest ? 1 : 0);
    while (pos < end) {
    const int64_t pg = pos / hout;
    const int32_t ha = static_cast<int32_t>(pos - pg * hout);
    const int32_t hb = static_cast<int32_t>(min(static_cast<int64_t>(min(hout, ha + tileRows)), ha + (end - pos)));
    pos += hb - ha;
    if constexpr (PERIODIC) {
        __syncthreads(); // the previous tile's entries are no longer read
        for (int32_t i = tid; i < hb - ha; i += nthreads) {
            int32_t lo, hi;
            float delta;
            LerpEntry(geomH, halfPixel, 0, ha + i, lo, hi, delta);
            rowT[i] = make_float4(__int_as_float(lo), __int_as_float(hi), delta, 0.0f);
        }
        __syncthreads();
    }
    // row entry of output row h of this tile
    auto rowEntry = [&](int32_t h, int32_t& lo, int32_t& hi, float& delta) {
        if constexpr (PERIODIC) {
            const float4 e = rowT[h - ha];
            lo = __float_as_int(e.x);
            hi = __float_as_int(e.y);
            delta = e.z;
        } else {
            lo = __ldg(th.lo + h);
            hi = __ldg(th.hi + h);
            delta = __ldg(th.delta + h);
        }
    };
    const int64_t p = pg * blockDim.y + threadIdx.y;
    if (p >= planes) {
        continue; // the barriers above are reached by every thread of the block in every tile
    }
    const int32_t groups = win / VI;
    const int32_t colThreads = blockDim.x, cg0 = threadIdx.x;
    // input and output may be views with N, C and H pitches (a dense tensor has those of its extents); W strides are 1
    const int64_t pn = PITCH ? p / outPitch.chan : 0;
    const T* xp = PITCH ? x + pn * inPitch.n + (p - pn * outPitch.chan) * inPitch.c : x + p * hin * static_cast<int64_t>(win);
    const int64_t inRow = PITCH ? inPitch.h : win;
    T* yp = PITCH ? y + pn * outPitch.n + (p - pn * outPitch.chan) * outPitch.c : y + p * hout * static_cast<int64_t>(wout);
    const int64_t outRow = PITCH ? outPitch.h : wout;
    for (int32_t g = cg0; g < groups; g += colThreads) {
        const int32_t c0 = g * VI;
        const int32_t cl = max(c0 - 1, 0), cr = min(c0 + VI, win - 1);
        float dx[PERIODIC ? 1 : VO], dx1[PERIODIC ? 1 : VO];
        if constexpr (!PERIODIC) {
#pragma unroll
            for (int k = 0; k < VO; ++k) {
                dx[k] = __ldg(tw.delta + c0 * 2 + k);
                dx1[k] = Sub(1.0f, dx[k]);
            }
        }
        // PERIODIC: only this thread's first output column can differ from the two repeating weights
        const float dxHead = c0 == 0 ? dxFirst : dxEven;
        const float dxHead1 = Sub(1.0f, dxHead), dxEven1 = Sub(1.0f, dxEven), dxOdd1 = Sub(1.0f, dxOdd);
        auto wR = [&](int k) { return PERIODIC ? (k == 0 ? dxHead : ((k & 1) ? dxOdd : dxEven)) : dx[PERIODIC ? 0 : k]; };
        auto wL = [&](int k) { return PERIODIC ? (k == 0 ? dxHead1 : ((k & 1) ? dxOdd1 : dxEven1)) : dx1[PERIODIC ? 0 : k]; };
        // QUEUE: the input rows this walk needs are lo[ha] .. hi[hb-1], in increasing order; they stream through
        // the thread's queue kW2QueueDepth rows ahead (one commit group per row, empty past the end).
        int32_t firstLo = 0, firstHi = 0, lastLo = 0, lastHi = 0;
        float unusedDelta = 0.0f;
        if (QUEUE) {
            rowEntry(ha, firstLo, firstHi, unusedDelta);
            rowEntry(hb - 1, lastLo, lastHi, unusedDelta);
        }
        const int32_t lastRow = lastHi;
        int32_t nextRow = firstLo; // next row the queue delivers
        int32_t issued = nextRow;                        // next row to start copying
        const T* issuePtr = xp + static_cast<int64_t>(nextRow) * inRow + c0;
        auto issue = [&]() {
            if (issued <= lastRow) {
                const int32_t slot = (issued & (kW2QueueDepth - 1)) * nthreads + tid;
                const T* xr = issuePtr;
                CpAsync16(qMid + slot, xr);
                if (c0 > 0) { // the word holding column c0-1 (4-byte aligned: c0 is a multiple of VI)
                    CpAsync4(qLeft + slot, xr - HE);
                }
                if (c0 + VI < win) {
                    CpAsync4(qRight + slot, xr + VI);
                }
            }
            ++issued;
            issuePtr += inRow;
            CpAsyncCommit();
        };
        if (QUEUE) {
#pragma unroll
            for (int d = 0; d < kW2QueueDepth; ++d) {
                issue();
            }
        }
        auto loadRow = [&](int32_t r, float (&h)[VO]) {
            const T* xr = xp + static_cast<int64_t>(r) * inRow;
            float v[VI + 2]; // columns c0-1 .. c0+VI
            if (QUEUE) {
                while (nextRow < r) { // rows the walk skips (down-scaling) are dropped
                    ++nextRow;
                    issue();
                }
                CpAsyncWait<kW2QueueDepth - 1>();
                const int32_t slot = (r & (kW2QueueDepth - 1)) * nthreads + tid;
                const uint4 raw = qMid[slot];
                float mid[VI];
                UnpackToF<T, VI>(reinterpret_cast<const Pack<T, VI>&>(raw), mid);
#pragma unroll
                for (int k = 0; k < VI; ++k) {
                    v[k + 1] = mid[k];
                }
                v[0] = v[1];
                v[VI + 1] = v[VI];
                if (c0 > 0) {
                    const uint32_t wl = qLeft[slot];
                    v[0] = DType<T>::ToF(reinterpret_cast<const T*>(&wl)[HE - 1]);
                }
                if (c0 + VI < win) {
                    const uint32_t wr = qRight[slot];
                    v[VI + 1] = DType<T>::ToF(reinterpret_cast<const T*>(&wr)[0]);
                }
                ++nextRow;
                issue();
            } else {
                v[0] = DType<T>::Load(xr + cl);
                float mid[VI];
                LoadPackLdg<T, VI>(xr + c0, mid);
#pragma unroll
                for (int k = 0; k < VI; ++k) {
                    v[k + 1] = mid[k];
                }
                v[VI + 1] = DType<T>::Load(xr + cr);
            }
#pragma unroll
            for (int j = 0; j < VI; ++j) {
                // outputs 2(c0+j) (taps c0+j-1, c0+j) and 2(c0+j)+1 (taps c0+j, c0+j+1)
                if constexpr (FUSE) {
                    h[2 * j] = fmaf(wR(2 * j), v[j + 1], Mul(wL(2 * j), v[j]));
                    h[2 * j + 1] = fmaf(wR(2 * j + 1), v[j + 2], Mul(wL(2 * j + 1), v[j + 1]));
                } else {
                    h[2 * j] = Add(Mul(wL(2 * j), v[j]), Mul(wR(2 * j), v[j + 1]));
                    h[2 * j + 1] = Add(Mul(wL(2 * j + 1), v[j + 1]), Mul(wR(2 * j + 1), v[j + 2]));
                }
            }
        };
        // Two row buffers; which of them holds the upper row alternates, so a row that moves from "lower" to "upper"
        // (every other output row when up-scaling) stays where it is. step() is the walk for one output row with
        // `up` as the upper and `dn` as the lower buffer and returns true when the two have traded places.
        float bufA[VO], bufB[VO];
        int32_t curTop = -1, curBot = -1;
        T* dst = yp + static_cast<int64_t>(ha) * outRow + c0 * 2;
        auto step = [&](int32_t h, float (&up)[VO], float (&dn)[VO]) -> bool {
            int32_t lo, hi;
            float dy;
            rowEntry(h, lo, hi, dy);
            if (lo == curBot && lo != curTop) { // the lower row becomes the upper one: trade places
                curTop = lo;
                if (hi == lo) {
#pragma unroll
                    for (int k = 0; k < VO; ++k) {
                        up[k] = dn[k];
                    }
                } else {
                    loadRow(hi, up);
                }
                curBot = hi;
                BlendStore<T, VO>(dst, dn, up, dy, wideStores != 0);
                dst += outRow;
                return true;
            }
            if (lo != curTop) {
                loadRow(lo, up);
                curTop = lo;
            }
            if (hi != curBot) {
                if (hi == curTop) {
#pragma unroll
                    for (int k = 0; k < VO; ++k) {
                        dn[k] = up[k];
                    }
                } else {
                    loadRow(hi, dn);
                }
                curBot = hi;
            }
            BlendStore<T, VO>(dst, up, dn, dy, wideStores != 0);
            dst += outRow;
            return false;
        };
        if constexpr (X2ROWS && PERIODIC) {
            auto put = [&](const float (&up)[VO], const float (&dn)[VO], int32_t h) {
                BlendStore<T, VO>(dst, up, dn, rowT[h - ha].z, wideStores != 0);
                dst += outRow;
            };
            int32_t h = ha, i = 0;
            if (h == 0) {
                loadRow(0, bufA);
                put(bufA, bufA, 0);
                h = 1;
            } else {
                i = (h - 1) >> 1;
                loadRow(i, bufA);
            }
            while (h < hb) { // bufA holds input row i; h is 2i + 1, or 2i + 2 where a tile starts inside a pair
                if (i == hin - 1) {
                    put(bufA, bufA, h);
                    break;
                }
                loadRow(i + 1, bufB);
                if (h == 2 * i + 1) {
                    put(bufA, bufB, h);
                    if (++h >= hb) {
                        break;
                    }
                }
                put(bufA, bufB, h);
                ++i;
                if (++h >= hb) {
                    break;
                }
                if (i == hin - 1) { // bufB holds input row i; h is 2i + 1
                    put(bufB, bufB, h);
                    break;
                }
                loadRow(i + 1, bufA);
                put(bufB, bufA, h);
                if (++h >= hb) {
                    break;
                }
                put(bufB, bufA, h);
                ++i;
                ++h;
            }
        } else {
        bool traded = false; // false: bufA is the upper row
        for (int32_t h = ha; h < hb; ++h) {
            const bool t = traded ? step(h, bufB, bufA) : step(h, bufA, bufB);
            traded ^= t;
        }
        }
        if (QUEUE) {
            CpAsyncWait<0>(); // nothing of this thread's queue is in flight when the next column group reuses it
        }
    }
    } // tiles of this block's run
}

// ---- backward row walk ---------------------------------------------------------------------------------------
// Combined weight with which grads index j feeds input index xcol: (lo == xcol ? 1-d : 0) + (hi == xcol ? d : 0).
__device__ __forceinline__ float CombinedWeight(const LerpAxis& t, int32_t j, int32_t xcol)
{
    const float d = __ldg(t.delta + j);
    float w = 0.0f;
    if (__ldg(t.lo + j) == xcol) {
        w = Sub(1.0f, d);
    }
    if (__ldg(t.hi + j) == xcol) {
        w = Add(w, d);
    }
    return w;
}

// A source j whose two taps fall on the same input index (lo == hi == xcol, at a clamped border) with a tap weight of
// exactly zero: the reference adds both products, so a non-finite grads value must still turn into NaN there
// although the combined weight is 1. Callers add one extra zero-weight product for such sources.
__device__ __forceinline__ bool HasZeroTwin(const LerpAxis& t, int32_t j, int32_t xcol)
{
    const float d = __ldg(t.delta + j);
    return __ldg(t.lo + j) == xcol && __ldg(t.hi + j) == xcol && (d == 0.0f || d == 1.0f);
}

// Vertical part of the walk, shared by the staged and the input-major kernels. `reduceRow(i, hp)` fills hp[] with the
// horizontally reduced grads row i for this thread's V grad_input columns. Rows [ya, yb) of grad_input are
// produced; grads rows are visited in increasing order and each contributes to rows lo[i] and hi[i] only.
template <typename TOut, int V, typename F>
__device__ __forceinline__ void WalkRows(TOut* dstBase, int32_t win, int32_t ya, int32_t yb, const LerpAxis& th,
                                         const RangeAxis& rh, F reduceRow)
{
    float accA[V], accB[V];
#pragma unroll
    for (int k = 0; k < V; ++k) {
        accA[k] = 0.0f;
        accB[k] = 0.0f;
    }
    int32_t cur = ya;
    TOut* dst = dstBase + static_cast<int64_t>(ya) * win;
    const int32_t is = __ldg(rh.start + ya), ie = max(is, __ldg(rh.end + yb - 1));
    for (int32_t i = is; i < ie; ++i) {
        const int32_t loY = __ldg(th.lo + i), hiY = __ldg(th.hi + i);
        const float dY = __ldg(th.delta + i);
        while (cur < loY && cur < yb) { // rows below lo[i] are complete
            StorePack<TOut, V>(dst, accA);
            dst += win;
#pragma unroll
            for (int k = 0; k < V; ++k) {
                accA[k] = accB[k];
                accB[k] = 0.0f;
            }
            ++cur;
        }
        if (cur >= yb) {
            break;
        }
        float hp[V];
        reduceRow(i, hp);
        const float wLo = Sub(1.0f, dY), wHi = dY;
        if (loY == cur) {
#pragma unroll
            for (int k = 0; k < V; ++k) {
                accA[k] = fmaf(wLo, hp[k], accA[k]);
            }
        } else if (loY == cur + 1) {
#pragma unroll
            for (int k = 0; k < V; ++k) {
                accB[k] = fmaf(wLo, hp[k], accB[k]);
            }
        }
        if (hiY == cur) {
#pragma unroll
            for (int k = 0; k < V; ++k) {
                accA[k] = fmaf(wHi, hp[k], accA[k]);
            }
        } else if (hiY == cur + 1 && cur + 1 < yb) {
#pragma unroll
            for (int k = 0; k < V; ++k) {
                accB[k] = fmaf(wHi, hp[k], accB[k]);
            }
        }
    }
    while (cur < yb) {
        StorePack<TOut, V>(dst, accA);
        dst += win;
#pragma unroll
        for (int k = 0; k < V; ++k) {
            accA[k] = accB[k];
            accB[k] = 0.0f;
        }
        ++cur;
    }
}

// ---- backward, NCHW, shared-memory staged ------------------------------------------------------------------------
// KW = compile-time bound on the number of grads columns feeding one grad_input column (the host checks it).
template <typename TIn, typename TOut, int V, int KW>
__global__ void __launch_bounds__(kThreads)
    BilinearBwdTileKernel(const TIn* __restrict__ go, TOut* __restrict__ gi, int64_t planes, int32_t hin, int32_t win,
                          int32_t hout, int32_t wout, LerpAxis th, LerpAxis tw, RangeAxis rh, RangeAxis rw,
                          int32_t tileRows, int32_t stageStride)
{
    extern __shared__ __align__(16) unsigned char smemRaw[];
    // block = (column threads, planes): the bands of blockDim.y planes are staged, `stageStride` bytes apart
    const int64_t pBase = static_cast<int64_t>(blockIdx.x) * blockDim.y;
    const int32_t np = static_cast<int32_t>(min(static_cast<int64_t>(blockDim.y), planes - pBase));
    const int32_t ya = blockIdx.y * tileRows, yb = min(hin, ya + tileRows);
    const int32_t r0 = __ldg(rh.start + ya);
    const int32_t r1 = max(r0, __ldg(rh.end + yb - 1));
    const int64_t planeElems = hout * static_cast<int64_t>(wout);
    const TIn* src = nullptr;
    for (int32_t pl = 0; pl < np; ++pl) {
        const TIn* staged = StageSpan<TIn>(go + (pBase + pl) * planeElems + static_cast<int64_t>(r0) * wout,
                                           static_cast<int64_t>(r1 - r0) * wout, smemRaw + pl * stageStride);
        if (pl == static_cast<int32_t>(threadIdx.y)) {
            src = staged;
        }
    }
    __syncthreads();
    if (static_cast<int32_t>(threadIdx.y) >= np) {
        return;
    }
    const int64_t p = pBase + threadIdx.y;
    const int32_t groups = win / V;
    const int32_t colThreads = blockDim.x, cg0 = threadIdx.x;
    TOut* gp = gi + p * hin * static_cast<int64_t>(win);
    for (int32_t g = cg0; g < groups; g += colThreads) {
        int32_t js[V], cnt[V];
        float wx[V][KW];
        uint32_t zeroTwins = 0; // bit k * KW + t: source js[k] + t adds one more zero-weight product to column k
#pragma unroll
        for (int k = 0; k < V; ++k) {
            const int32_t xcol = g * V + k;
            js[k] = __ldg(rw.start + xcol);
            cnt[k] = __ldg(rw.end + xcol) - js[k];
#pragma unroll
            for (int t = 0; t < KW; ++t) {
                wx[k][t] = t < cnt[k] ? CombinedWeight(tw, js[k] + t, xcol) : 0.0f;
                if (t < cnt[k] && HasZeroTwin(tw, js[k] + t, xcol)) {
                    zeroTwins |= 1u << (k * KW + t);
                }
            }
        }
        WalkRows<TOut, V>(gp + g * V, win, ya, yb, th, rh, [&](int32_t i, float (&hp)[V]) {
            const TIn* row = src + (i - r0) * wout;
#pragma unroll
            for (int k = 0; k < V; ++k) {
                float a = 0.0f;
#pragma unroll
                for (int t = 0; t < KW; ++t) {
                    // taps past the run are not read (they may lie outside the row, or hold Inf / NaN)
                    const float v = (t < cnt[k]) ? DType<TIn>::ToF(row[js[k] + t]) : 0.0f;
                    a = fmaf(wx[k][t], v, a);
                }
                hp[k] = a;
            }
            if (zeroTwins != 0) { // only threads at a clamped border
#pragma unroll
                for (int k = 0; k < V; ++k) {
#pragma unroll
                    for (int t = 0; t < KW; ++t) {
                        if (zeroTwins & (1u << (k * KW + t))) {
                            hp[k] = fmaf(0.0f, DType<TIn>::ToF(row[js[k] + t]), hp[k]);
                        }
                    }
                }
            }
        });
    }
}

// ---- backward, NCHW, grads width = 2 x grad_input width, input-major ------------------------------------------------
// The host has verified the column pattern: grad_input column x is fed by grads columns 2x-1 .. 2x+2 (clipped to
// the row). A thread owns four grad_input columns x0..x0+3 and reads grads columns 2*x0-1 .. 2*x0+8 of each row:
// one 16-byte (fp16/bf16) or two 16-byte (fp32) vectors plus one neighbour on each side.
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(kThreads)
    BilinearBwdW2Kernel(const TIn* __restrict__ go, TOut* __restrict__ gi, int64_t planes, int32_t hin, int32_t win,
                        int32_t hout, LerpAxis th, LerpAxis tw, RangeAxis rh, int32_t tileRows)
{
    constexpr int V = 4, VG = 8;
    const int32_t wout = 2 * win;
    // block = (column threads, planes): every thread of a block walks the same rows, so the row logic is uniform
    const int64_t p = static_cast<int64_t>(blockIdx.x) * blockDim.y + threadIdx.y;
    if (p >= planes) {
        return;
    }
    const int32_t ya = blockIdx.y * tileRows, yb = min(hin, ya + tileRows);
    const int32_t groups = win / V;
    const int32_t colThreads = blockDim.x, cg0 = threadIdx.x;
    const TIn* gp = go + p * hout * static_cast<int64_t>(wout);
    TOut* op = gi + p * hin * static_cast<int64_t>(win);
    for (int32_t g = cg0; g < groups; g += colThreads) {
        const int32_t x0 = g * V, j0 = 2 * x0;
        const bool hasLeft = j0 > 0, hasRight = j0 + VG < wout;
        // wx[k][t]: weight of grads column 2*(x0+k) - 1 + t for grad_input column x0+k (0 outside the row)
        float wx[V][4];
        uint32_t zeroTwins = 0; // bit k * 4 + t: that source adds one more zero-weight product (clamped border)
#pragma unroll
        for (int k = 0; k < V; ++k) {
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const int32_t j = j0 + 2 * k - 1 + t;
                wx[k][t] = (j >= 0 && j < wout) ? CombinedWeight(tw, j, x0 + k) : 0.0f;
                if (j >= 0 && j < wout && HasZeroTwin(tw, j, x0 + k)) {
                    zeroTwins |= 1u << (k * 4 + t);
                }
            }
        }
        // Column 1 has one more source: grads column 0 is clamped to input column 0 with delta 0, and the
        // reference still adds its (zero-weight) "hi" product to column 1.
        const bool extra = x0 == 0 && win > 1;
        const float wExtra = extra ? CombinedWeight(tw, 0, 1) : 0.0f;
        WalkRows<TOut, V>(op + x0, win, ya, yb, th, rh, [&](int32_t i, float (&hp)[V]) {
            const TIn* row = gp + static_cast<int64_t>(i) * wout + j0;
            float v[VG + 2]; // grads columns j0-1 .. j0+8; neighbours outside the row read as 0 (weight 0)
            v[0] = hasLeft ? DType<TIn>::Load(row - 1) : 0.0f;
            float mid[VG];
            if constexpr (sizeof(TIn) == 2) {
                LoadPackLdg<TIn, VG>(row, mid);
            } else {
                float a[4], b[4];
                LoadPackLdg<TIn, 4>(row, a);
                LoadPackLdg<TIn, 4>(row + 4, b);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    mid[k] = a[k];
                    mid[k + 4] = b[k];
                }
            }
#pragma unroll
            for (int k = 0; k < VG; ++k) {
                v[k + 1] = mid[k];
            }
            v[VG + 1] = hasRight ? DType<TIn>::Load(row + VG) : 0.0f;
#pragma unroll
            for (int k = 0; k < V; ++k) {
                float a = 0.0f;
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    a = fmaf(wx[k][t], v[2 * k + t], a);
                }
                hp[k] = a;
            }
            if (extra) {
                hp[1] = fmaf(wExtra, v[1], hp[1]);
            }
            if (zeroTwins != 0) { // only threads at a clamped border (align_corners)
#pragma unroll
                for (int k = 0; k < V; ++k) {
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        if (zeroTwins & (1u << (k * 4 + t))) {
                            hp[k] = fmaf(0.0f, v[2 * k + t], hp[k]);
                        }
                    }
                }
            }
        });
    }
}

// ---- backward, NCHW, grads = 2 x grad_input on both axes, input-major ---------------------------------------------
// The host has verified the pattern on both axes: grads row i feeds grad_input rows lo[i] = max((i-1)>>1, 0) and
// hi[i] (lo[i] + 1 clipped to the plane; row 0 feeds rows 0 and 1), and the same for columns. A thread owns four
// grad_input columns and walks down the grads rows that feed its tile of grad_input rows. Every grads row is reduced
// horizontally once and added into the (at most two) open grad_input rows, in increasing grads-row order and lower
// tap first, which is the order of the reference's scatter loop; zero-weight taps at clamped borders are real
// products here, so NaN / Inf propagate as they do there.
// The grads rows a thread consumes form a plain stream. The thread copies its own piece of each row (its eight
// columns plus one neighbour on each side) with cp.async into a private shared-memory queue kX2Depth rows ahead: the
// walk is a serial chain per thread, so what bounds it is the number of bytes in flight, and a queue in shared
// memory holds several times what the registers could.
// What a grads row does to the open rows (its two weights, which of the open rows they go to, how many finished rows
// to store first) is the same for every thread: it is evaluated once per block into shared memory.
// rows in flight per thread (a power of two: the slot of a stream element is a mask away); the same bytes for both widths
constexpr int X2Depth(int cols) { return cols == 8 ? 4 : 8; }

inline size_t X2SmemBytes(int32_t tileRows, int32_t threads, int elemSize, int cols)
{
    const size_t recs = static_cast<size_t>(2 * tileRows + 4) * 16; // one 16-byte record per grads row of the tile
    return recs + static_cast<size_t>(X2Depth(cols)) * threads * (2 * cols * elemSize + 8);
}

// TWINS: the column table holds clamped-border sources whose two taps fall on one index with a weight of exactly
// zero (align_corners); the host knows from its copy of the tables, and only then the extra zero-weight products of
// the horizontal reduction are compiled in.
// V: grad_input columns per thread (4, or 8 with PERIODIC and 16-bit tensors).
// PERIODIC: the host has checked that the four column weights of a grad_input column are the same for every column
// but the first and the last of a row; they arrive as scalars (pw0..pw3) and only the two border weights are read
// from the table, which frees the registers a second group of four columns needs.
template <typename TIn, typename TOut, bool TWINS, int V, bool PERIODIC, bool PITCH = false>
__global__ void __launch_bounds__(kW2Threads, 5)
    BilinearBwdX2Kernel(const TIn* __restrict__ go, TOut* __restrict__ gi, int64_t planes, int32_t hin, int32_t win,
                        LerpAxis th, LerpAxis tw, RangeAxis rh, int32_t tileRows, float pw0, float pw1, float pw2,
                        float pw3, AxisGeom geomH, AxisGeom geomW, int32_t halfPixel, int32_t start1,
                        ViewStrides gradsPitch)
{
    // PERIODIC reads no table: row entries and the three border weights are evaluated from the geometry (LerpEntry is
    // what the table kernel runs, so the bits are the same), and the first / last grads row of a tile follow from
    // the 2x pattern the host has verified (start1: where the range of grad_input row 1 starts, 0 or 1).
    // table entry of grads index i on the row (axis 0) or column axis
    auto entry = [&](int axis, int32_t i, int32_t& lo, int32_t& hi, float& d) {
        if constexpr (PERIODIC) {
            LerpEntry(axis == 0 ? geomH : geomW, halfPixel, 1, i, lo, hi, d);
        } else {
            const LerpAxis& t = axis == 0 ? th : tw;
            lo = __ldg(t.lo + i);
            hi = __ldg(t.hi + i);
            d = __ldg(t.delta + i);
        }
    };
    // weight with which grads column j feeds grad_input column xcol (as CombinedWeight does from the table)
    auto colWeight = [&](int32_t j, int32_t xcol) {
        int32_t lo, hi;
        float d;
        entry(1, j, lo, hi, d);
        float w = 0.0f;
        if (lo == xcol) {
            w = Sub(1.0f, d);
        }
        if (hi == xcol) {
            w = Add(w, d);
        }
        return w;
    };
    constexpr int VG = 2 * V;
    constexpr int kX2Depth = X2Depth(V);
    constexpr int NM = VG * sizeof(TIn) / 16; // 16-byte vectors holding grads columns j0 .. j0+VG-1
    constexpr int HE = 4 / sizeof(TIn);       // elements in a 4-byte neighbour word
    // bits of a row record
    constexpr int kLoA = 1, kHiA = 4, kHiB = 8, kFlushShift = 4;
    extern __shared__ __align__(16) unsigned char x2Smem[];
    float4* rowRec = reinterpret_cast<float4*>(x2Smem); // per grads row of the tile: {1-d, d, bits, -}
    const int32_t wout = 2 * win;
    const int32_t tid = threadIdx.y * blockDim.x + threadIdx.x, nthreads = blockDim.x * blockDim.y;
    // queue: [kX2Depth][nthreads] entries of NM 16-byte vectors, then [kX2Depth][nthreads] {left, right} word pairs.
    // A thread's vectors stay next to each other: spreading them over separate planes (no bank conflicts) doubled
    // the L2 requests of the copies and was slower (85 us against 67 us on fp16 32x256x112x112 -> 56x56).
    unsigned char* qBase = x2Smem + static_cast<size_t>(2 * tileRows + 4) * 16;
    const uint32_t strideMid = static_cast<uint32_t>(nthreads) * 16 * NM; // bytes between slots
    unsigned char* midP = qBase + static_cast<size_t>(tid) * 16 * NM;
    unsigned char* lrP = qBase + static_cast<size_t>(kX2Depth) * strideMid + static_cast<size_t>(tid) * 8;
    // The grad_input rows of all plane groups form one sequence (group-major); the blocks cut it into gridDim.x equal
    // runs, so that one wave of resident blocks finishes together whatever the number of planes. A run is walked as
    // tiles: its pieces of consecutive plane groups, none taller than tileRows.
    const int64_t planeGroups = (planes + blockDim.y - 1) / blockDim.y;
    const int64_t totalRows = planeGroups * hin;
    const int64_t share = totalRows / gridDim.x, rest = totalRows - share * gridDim.x; // the first `rest` runs get one more
    int64_t pos = share * blockIdx.x + min(static_cast<int64_t>(blockIdx.x), rest);
    const int64_t end = pos + share + (blockIdx.x < rest ? 1 : 0);
    while (pos < end) {
    const int64_t pg = pos / hin;
    const int32_t ya = static_cast<int32_t>(pos - pg * hin);
    const int32_t yb = static_cast<int32_t>(min(static_cast<int64_t>(min(hin, ya + tileRows)), ya + (end - pos)));
    pos += yb - ya;
    // grads rows [first, first + count) feed grad_input rows [ya, yb)
    const int32_t first = PERIODIC ? (ya == 1 ? start1 : max(2 * ya - 1, 0)) : __ldg(rh.start + ya);
    const int32_t last = PERIODIC ? min(2 * (yb - 1) + 3, 2 * hin) : __ldg(rh.end + yb - 1);
    const int32_t count = min(max(first, last) - first, 2 * tileRows + 4);
    __syncthreads(); // the previous tile's records are no longer read
    for (int32_t n = tid; n < count; n += nthreads) {
        const int32_t i = first + n;
        int32_t lo, hi, loPrev = 0, hiPrev;
        float d, dPrev;
        entry(0, i, lo, hi, d);
        if (n > 0) {
            entry(0, i - 1, loPrev, hiPrev, dPrev);
        }
        // the older open row when row i is added: rows below lo[i] are complete
        const int32_t cur = max(ya, lo);
        const int32_t prev = n > 0 ? max(ya, loPrev) : ya;
        int32_t bits = (cur - prev) << kFlushShift;
        bits |= (lo == cur) ? kLoA : 0;
        bits |= (hi == cur) ? kHiA : 0;
        bits |= (hi == cur + 1 && hi < yb) ? kHiB : 0;
        rowRec[n] = make_float4(Sub(1.0f, d), d, __int_as_float(bits), 0.0f);
    }
    __syncthreads();
    const int64_t p = pg * blockDim.y + threadIdx.y;
    if (p >= planes) {
        continue; // the barriers above are reached by every thread of the block in every tile
    }
    const int32_t groups = win / V;
    // grad_output may be a view with N, C and H pitches (a dense tensor has those of its extents); its W stride is 1
    const int64_t pn = PITCH ? p / gradsPitch.chan : 0;
    const TIn* gp = PITCH ? go + pn * gradsPitch.n + (p - pn * gradsPitch.chan) * gradsPitch.c
                          : go + p * (2 * static_cast<int64_t>(hin)) * wout;
    const int64_t gradsRow = PITCH ? gradsPitch.h : wout;
    TOut* op = gi + p * hin * static_cast<int64_t>(win);
    for (int32_t g = threadIdx.x; g < groups; g += blockDim.x) {
        const int32_t x0 = g * V, j0 = 2 * x0;
        const bool hasLeft = j0 > 0, hasRight = j0 + VG < wout;
        // wx[k][t]: weight of grads column 2*(x0+k) - 1 + t for grad_input column x0+k (0 outside the row)
        float wx[PERIODIC ? 1 : V][4];
        uint32_t zeroTwins = 0; // bit k * 4 + t: that source adds one more zero-weight product (clamped border)
        if constexpr (!PERIODIC) {
#pragma unroll
            for (int k = 0; k < V; ++k) {
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const int32_t j = j0 + 2 * k - 1 + t;
                    wx[k][t] = (j >= 0 && j < wout) ? CombinedWeight(tw, j, x0 + k) : 0.0f;
                    if (TWINS && j >= 0 && j < wout && HasZeroTwin(tw, j, x0 + k)) {
                        zeroTwins |= 1u << (k * 4 + t);
                    }
                }
            }
        }
        // PERIODIC: grads column 0 feeds column 0 and grads column wout-1 feeds column win-1 with their own weights;
        // the taps that fall outside the row multiply a zero
        const float wHead = (PERIODIC && x0 == 0) ? colWeight(0, 0) : pw1;
        const float wTail = (PERIODIC && x0 + V == win) ? colWeight(wout - 1, win - 1) : pw2;
        auto weight = [&](int k, int t) {
            if constexpr (PERIODIC) {
                return (k == 0 && t == 1)
                           ? wHead
                           : ((k == V - 1 && t == 2) ? wTail : (t == 0 ? pw0 : (t == 1 ? pw1 : (t == 2 ? pw2 : pw3))));
            } else {
                return wx[k][t];
            }
        };
        const bool extra = x0 == 0 && win > 1; // column 1 also takes grads column 0 (zero weight), as for rows
        const float wExtra = extra ? colWeight(0, 1) : 0.0f;
        // one commit group per stream element (empty past the end); elements are issued in order, so the source
        // advances by one row per call
        const TIn* issueRow = gp + static_cast<int64_t>(first) * gradsRow + j0;
        int32_t issueLeft = count;
        // The neighbour columns j0-1 and j0+VG are the last / first column of the threads to the left and right, whose
        // queue slots lie next to this thread's. When that thread is a lane of the same warp (same plane row, same
        // stream element at the same time) its copy is read instead of copying the word again: the separate 4-byte
        // copies made every 32-byte sector of grads travel from L2 three times (ncu: 3.4 x the tensor on the L2-to-SM
        // path, which is what bounded the kernel). Only lanes at a warp edge still copy their own neighbour word.
        const unsigned warpMask = __activemask();
        const int32_t laneId = tid & 31;
        const bool leftShared = hasLeft && threadIdx.x > 0 && laneId > 0;
        const bool rightShared = hasRight && threadIdx.x + 1 < blockDim.x && laneId < 31 && g + 1 < groups;
        auto issue = [&](unsigned char* pm, unsigned char* plr) {
            if (issueLeft > 0) {
#pragma unroll
                for (int m = 0; m < NM; ++m) {
                    CpAsync16(pm + 16 * m, reinterpret_cast<const uint4*>(issueRow) + m);
                }
                if (hasLeft && !leftShared) { // the word holding column j0-1 (4-byte aligned: j0 is a multiple of 8)
                    CpAsync4(plr, issueRow - HE);
                }
                if (hasRight && !rightShared) {
                    CpAsync4(plr + 4, issueRow + VG);
                }
            }
            issueRow += gradsRow;
            --issueLeft;
            CpAsyncCommit();
        };
        // Reduced row n of the stream. Waits until all but the newest kX2Depth-1 groups have landed, i.e. until
        // element n has, then refills its slot with element n + kX2Depth.
        auto take = [&](int32_t n, float (&hp)[V]) {
            CpAsyncWait<kX2Depth - 1>();
            __syncwarp(warpMask); // every lane's copy of element n has landed: the neighbours' slots may be read
            const uint32_t off = static_cast<uint32_t>(n & (kX2Depth - 1)) * strideMid;
            unsigned char* pm = midP + off;
            unsigned char* plr = lrP + off / (2 * NM);
            uint4 mid[NM];
#pragma unroll
            for (int m = 0; m < NM; ++m) {
                mid[m] = reinterpret_cast<const uint4*>(pm)[m];
            }
            uint2 lr = *reinterpret_cast<const uint2*>(plr);
            if (leftShared) {
                lr.x = *reinterpret_cast<const uint32_t*>(pm - 4);        // last word of the left neighbour's slot
            }
            if (rightShared) {
                lr.y = *reinterpret_cast<const uint32_t*>(pm + 16 * NM);  // first word of the right neighbour's slot
            }
            __syncwarp(warpMask); // all lanes have read before any slot is refilled
            issue(pm, plr);
            float v[VG + 2]; // grads columns j0-1 .. j0+8
            {
                float all[VG];
                UnpackToF<TIn, VG>(*reinterpret_cast<const Pack<TIn, VG>*>(mid), all);
#pragma unroll
                for (int k = 0; k < VG; ++k) {
                    v[k + 1] = all[k];
                }
            }
            // the neighbour words are not written (and not read as numbers) where the row ends
            v[0] = hasLeft ? DType<TIn>::ToF(reinterpret_cast<const TIn*>(&lr.x)[HE - 1]) : 0.0f;
            v[VG + 1] = hasRight ? DType<TIn>::ToF(reinterpret_cast<const TIn*>(&lr.y)[0]) : 0.0f;
#pragma unroll
            for (int k = 0; k < V; ++k) {
                float a = 0.0f;
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    a = fmaf(weight(k, t), v[2 * k + t], a);
                }
                hp[k] = a;
            }
            if (extra) {
                hp[1] = fmaf(wExtra, v[1], hp[1]);
            }
            if (TWINS && zeroTwins != 0) { // only threads at a clamped border (align_corners)
#pragma unroll
                for (int k = 0; k < V; ++k) {
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        if (zeroTwins & (1u << (k * 4 + t))) {
                            hp[k] = fmaf(0.0f, v[2 * k + t], hp[k]);
                        }
                    }
                }
            }
        };
#pragma unroll
        for (int n = 0; n < kX2Depth; ++n) {
            issue(midP + n * strideMid, lrP + n * (strideMid / (2 * NM)));
        }
        float accA[V], accB[V]; // rows cur and cur + 1
#pragma unroll
        for (int k = 0; k < V; ++k) {
            accA[k] = 0.0f;
            accB[k] = 0.0f;
        }
        int32_t cur = ya;
        TOut* dst = op + static_cast<int64_t>(ya) * win + x0;
        auto flush = [&]() {
            StorePack<TOut, V>(dst, accA);
            dst += win;
            ++cur;
#pragma unroll
            for (int k = 0; k < V; ++k) {
                accA[k] = accB[k];
                accB[k] = 0.0f;
            }
        };
        for (int32_t n = 0; n < count; ++n) {
            float hp[V];
            take(n, hp);
            const float4 rec = rowRec[n];
            const int32_t bits = __float_as_int(rec.z);
            for (int32_t f = bits >> kFlushShift; f > 0; --f) { // uniform over the block
                flush();
            }
            if ((bits & 15) == (kLoA | kHiB)) { // the interior case
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    accA[k] = fmaf(rec.x, hp[k], accA[k]);
                    accB[k] = fmaf(rec.y, hp[k], accB[k]);
                }
            } else {
                if (bits & kLoA) {
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        accA[k] = fmaf(rec.x, hp[k], accA[k]);
                    }
                }
                if (bits & kHiA) {
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        accA[k] = fmaf(rec.y, hp[k], accA[k]);
                    }
                }
                if (bits & kHiB) {
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        accB[k] = fmaf(rec.y, hp[k], accB[k]);
                    }
                }
            }
        }
        while (cur < yb) {
            flush();
        }
        CpAsyncWait<0>(); // nothing of this thread's queue is in flight when the next column group reuses it
    }
    } // tiles of this block's run
}

// ---- forward, NHWC ----------------------------------------------------------------------------------------
// A thread owns one vector of V channels of one output column (n, w) and walks down the output rows [h0, h1) of a
// row chunk. Its column taps (wl, wh, dx) are fixed, so it keeps the horizontally interpolated values of the two
// input rows in use (a: row ia, b: row ib) in registers; moving to the next output row reuses them when the row
// taps stay or shift by one, which for up-scaling is most of the time: about in/out vector loads and
// 3 * in/out + 3 fp32 operations per output element instead of 4 loads and 9 operations. The expression tree per
// element is the reference's, (1-dy) * ((1-dx) * TL + dx * TR) + dy * ((1-dx) * BL + dx * BR), unchanged.
// Consecutive threads hold consecutive channel vectors, then consecutive columns: every load and store of a warp
// is one contiguous run, and neighbouring columns find their shared input pixels in L1.
// QUEUE (16-byte channel vectors): the two pixels a thread needs of every input row stream through a per-thread
// cp.async queue kFwdQueueDepth rows ahead; without it the walk exposes one memory latency per new input row.
// FUSE (16-bit T): the host has checked that every column weight times any value of T is exact in fp32, so the
// horizontal interpolation uses one fused multiply-add: same bits, one instruction fewer.
// X2ROWS (with QUEUE, one row chunk): the host has checked that the row table is the 2x pattern; the walk then takes
// one new input row per two output rows in a straight line (no row indices, no comparisons, no copies between the
// two row buffers: the loop body is written twice with the buffers trading places). Same expressions, same bits.
template <typename T, int V, bool QUEUE, bool FUSE = false, bool X2ROWS = false>
__global__ void __launch_bounds__(kThreads)
    BilinearFwdNHWCKernel(const T* __restrict__ x, T* __restrict__ y, int32_t c, int32_t hin, int32_t win,
                          int32_t hout, int32_t wout, LerpAxis th, LerpAxis tw, int32_t rows, int32_t rowChunks,
                          int64_t walkers)
{
    extern __shared__ __align__(16) unsigned char nhwcQueue[];
    uint4* qL = reinterpret_cast<uint4*>(nhwcQueue);                 // [depth][blockDim.x] left pixel
    uint4* qR = qL + static_cast<size_t>(kFwdQueueDepth) * blockDim.x; // [depth][blockDim.x] right pixel
    const int32_t groups = c / V;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t total = walkers * rowChunks;
    for (int64_t id = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; id < total; id += stride) {
        const int64_t chunk = id / walkers; // chunk-major: a block stays inside one row chunk
        const int64_t wk = id - chunk * walkers;
        const int64_t col = wk / groups;
        const int32_t g = static_cast<int32_t>(wk - col * groups);
        const int64_t n = col / wout;
        const int32_t w = static_cast<int32_t>(col - n * wout);
        int32_t h0 = static_cast<int32_t>(chunk) * rows;
        const int32_t h1 = min(hout, h0 + rows);
        // X2ROWS: `rows` counts steps (a step = one new input row = two output rows); this walker takes the steps
        // [sA, sB), with output row 0 if it starts at step 0 and the last output row if it ends at the last step
        const int32_t sA = static_cast<int32_t>(chunk) * rows, sB = min(sA + rows, hin - 1);
        if constexpr (X2ROWS) {
            h0 = sA == 0 ? 0 : 2 * sA + 1;
        }
        const int32_t wl = __ldg(tw.lo + w), wh = __ldg(tw.hi + w);
        const float dx = __ldg(tw.delta + w), dx1 = Sub(1.0f, dx);
        const int64_t rowStride = static_cast<int64_t>(win) * c;
        const T* xl = x + n * hin * rowStride + static_cast<int64_t>(wl) * c + g * V;
        const T* xr = x + n * hin * rowStride + static_cast<int64_t>(wh) * c + g * V;
        T* yp = y + ((n * hout + h0) * wout + w) * c + static_cast<int64_t>(g) * V;
        const int64_t outStride = static_cast<int64_t>(wout) * c;
        float a[V], b[V];
        int32_t ia = -1, ib = -1;
        // QUEUE: rows lo[h0] .. hi[h1-1] are needed in increasing order
        const int32_t lastRow = X2ROWS ? sB : (QUEUE ? __ldg(th.hi + h1 - 1) : 0);
        int32_t nextRow = X2ROWS ? sA : (QUEUE ? __ldg(th.lo + h0) : 0), issued = nextRow;
        const T* issueL = xl + nextRow * rowStride; // row `issued` of the left / right pixel
        const T* issueR = xr + nextRow * rowStride;
        auto issue = [&]() {
            if (issued <= lastRow) {
                const int32_t slot = (issued & (kFwdQueueDepth - 1)) * blockDim.x + threadIdx.x;
                CpAsync16(qL + slot, issueL);
                CpAsync16(qR + slot, issueR);
            }
            ++issued;
            issueL += rowStride;
            issueR += rowStride;
            CpAsyncCommit();
        };
        if (QUEUE) {
#pragma unroll
            for (int d = 0; d < kFwdQueueDepth; ++d) {
                issue();
            }
        }
        auto hrow = [&](int32_t r, float (&dst)[V]) {
            float l[V], rr[V];
            if (QUEUE) {
                while (nextRow < r) { // rows the walk skips (down-scaling) are dropped
                    ++nextRow;
                    issue();
                }
                CpAsyncWait<kFwdQueueDepth - 1>();
                const int32_t slot = (r & (kFwdQueueDepth - 1)) * blockDim.x + threadIdx.x;
                const uint4 rawL = qL[slot], rawR = qR[slot];
                UnpackToF<T, V>(reinterpret_cast<const Pack<T, V>&>(rawL), l);
                UnpackToF<T, V>(reinterpret_cast<const Pack<T, V>&>(rawR), rr);
                ++nextRow;
                issue();
            } else {
                LoadPackLdg<T, V>(xl + r * rowStride, l);
                LoadPackLdg<T, V>(xr + r * rowStride, rr);
            }
            if constexpr (V % 2 == 0) {
                // two channels per instruction; each half keeps the scalar form's products and its one rounded sum
                const F2 DX = MakeF2(dx, dx), DX1 = MakeF2(dx1, dx1);
#pragma unroll
                for (int k = 0; k < V; k += 2) {
                    const F2 left = Mul2(DX1, MakeF2(l[k], l[k + 1])), right = MakeF2(rr[k], rr[k + 1]);
                    SplitF2(FUSE ? Fma2(DX, right, left) : AddProduct2(Mul2(DX, right), left), dst[k], dst[k + 1]);
                }
            } else {
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    dst[k] = FUSE ? fmaf(dx, rr[k], Mul(dx1, l[k])) : Add(Mul(dx1, l[k]), Mul(dx, rr[k]));
                }
            }
        };
        if constexpr (X2ROWS && QUEUE) {
            auto emit = [&](const float (&up)[V], const float (&dn)[V], int32_t h) {
                const float dy = __ldg(th.delta + h), dy1 = Sub(1.0f, dy);
                float out[V];
                if constexpr (V % 2 == 0) {
                    const F2 DY = MakeF2(dy, dy), DY1 = MakeF2(dy1, dy1);
#pragma unroll
                    for (int k = 0; k < V; k += 2) {
                        SplitF2(AddProduct2(Mul2(DY, MakeF2(dn[k], dn[k + 1])), Mul2(DY1, MakeF2(up[k], up[k + 1]))),
                                out[k], out[k + 1]);
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        out[k] = Add(Mul(dy1, up[k]), Mul(dy, dn[k]));
                    }
                }
                StorePack<T, V>(yp, out);
                yp += outStride;
            };
            hrow(sA, a);
            if (sA == 0) {
                emit(a, a, 0);
            }
            int32_t i = sA;
            for (; i + 2 <= sB; i += 2) {
                hrow(i + 1, b);
                emit(a, b, 2 * i + 1);
                emit(a, b, 2 * i + 2);
                hrow(i + 2, a);
                emit(b, a, 2 * i + 3);
                emit(b, a, 2 * i + 4);
            }
            if (i < sB) {
                hrow(i + 1, b);
                emit(a, b, 2 * i + 1);
                emit(a, b, 2 * i + 2);
                if (sB == hin - 1) {
                    emit(b, b, hout - 1);
                }
            } else if (sB == hin - 1) {
                emit(a, a, hout - 1);
            }
            CpAsyncWait<0>();
            continue;
        }
        for (int32_t h = h0; h < h1; ++h) {
            const int32_t hl = __ldg(th.lo + h), hh = __ldg(th.hi + h);
            const float dy = __ldg(th.delta + h), dy1 = Sub(1.0f, dy);
            if (hl != ia) {
                if (hl == ib) {
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        a[k] = b[k];
                    }
                } else {
                    hrow(hl, a);
                }
                ia = hl;
            }
            if (hh != ib) {
                if (hh == ia) {
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        b[k] = a[k];
                    }
                } else {
                    hrow(hh, b);
                }
                ib = hh;
            }
            float out[V];
            if constexpr (V % 2 == 0) {
                const F2 DY = MakeF2(dy, dy), DY1 = MakeF2(dy1, dy1);
#pragma unroll
                for (int k = 0; k < V; k += 2) {
                    SplitF2(AddProduct2(Mul2(DY, MakeF2(b[k], b[k + 1])), Mul2(DY1, MakeF2(a[k], a[k + 1]))), out[k],
                            out[k + 1]);
                }
            } else {
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    out[k] = Add(Mul(dy1, a[k]), Mul(dy, b[k]));
                }
            }
            StorePack<T, V>(yp, out);
            yp += outStride;
        }
        if (QUEUE) {
            CpAsyncWait<0>(); // the queue is empty before the thread takes another walker
        }
    }
}

// ---- backward, gather ---------------------------------------------------------------------------------------
// Adds to acc what the serial scatter would add to destination (y, x) from source (i, j), in its order
// TL, TR, BL, BR (resize_bilinear_v2_grad_simt.h:147-150): weights (dx1*dy1), (dx*dy1), (dx1*dy), (dx*dy) times g.
__device__ __forceinline__ float GatherTap(float acc, float g, int32_t y, int32_t x, int32_t loY, int32_t hiY,
                                           float dY, int32_t loX, int32_t hiX, float dX)
{
    const float dY1 = Sub(1.0f, dY), dX1 = Sub(1.0f, dX);
    if (loY == y) {
        if (loX == x) {
            acc = Add(acc, Mul(Mul(dX1, dY1), g));
        }
        if (hiX == x) {
            acc = Add(acc, Mul(Mul(dX, dY1), g));
        }
    }
    if (hiY == y) {
        if (loX == x) {
            acc = Add(acc, Mul(Mul(dX1, dY), g));
        }
        if (hiX == x) {
            acc = Add(acc, Mul(Mul(dX, dY), g));
        }
    }
    return acc;
}

template <typename TIn, typename TOut, int V>
__global__ void __launch_bounds__(kThreads)
    BilinearBwdGatherNCHWKernel(const TIn* __restrict__ go, TOut* __restrict__ gi, int32_t hin, int32_t win,
                                int32_t hout, int32_t wout, LerpAxis th, LerpAxis tw, RangeAxis rh, RangeAxis rw,
                                int64_t totalGroups)
{
    const int32_t groups = win / V;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; gid < totalGroups; gid += stride) {
        const int64_t row = gid / groups;
        const int32_t g = static_cast<int32_t>(gid - row * groups);
        const int64_t p = row / hin;
        const int32_t y = static_cast<int32_t>(row - p * hin);
        const int32_t is = __ldg(rh.start + y), ie = __ldg(rh.end + y);
        int32_t js[V], je[V];
        float acc[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            js[k] = __ldg(rw.start + g * V + k);
            je[k] = __ldg(rw.end + g * V + k);
            acc[k] = 0.0f;
        }
        const TIn* gp = go + p * hout * static_cast<int64_t>(wout);
        for (int32_t i = is; i < ie; ++i) {
            const int32_t loY = __ldg(th.lo + i), hiY = __ldg(th.hi + i);
            const float dY = __ldg(th.delta + i);
            const TIn* gr = gp + static_cast<int64_t>(i) * wout;
#pragma unroll
            for (int k = 0; k < V; ++k) {
                const int32_t x = g * V + k;
                for (int32_t j = js[k]; j < je[k]; ++j) {
                    acc[k] = GatherTap(acc[k], DType<TIn>::Load(gr + j), y, x, loY, hiY, dY, __ldg(tw.lo + j),
                                       __ldg(tw.hi + j), __ldg(tw.delta + j));
                }
            }
        }
        StorePack<TOut, V>(gi + row * win + static_cast<int64_t>(g) * V, acc);
    }
}

template <typename TIn, typename TOut, int V>
__global__ void __launch_bounds__(kThreads)
    BilinearBwdGatherNHWCKernel(const TIn* __restrict__ go, TOut* __restrict__ gi, int32_t c, int32_t hin,
                                int32_t win, int32_t hout, int32_t wout, LerpAxis th, LerpAxis tw, RangeAxis rh,
                                RangeAxis rw, int64_t totalGroups)
{
    const int32_t groups = c / V;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; gid < totalGroups; gid += stride) {
        const int64_t pix = gid / groups;
        const int32_t g = static_cast<int32_t>(gid - pix * groups);
        const int64_t nh = pix / win;
        const int32_t x = static_cast<int32_t>(pix - nh * win);
        const int64_t n = nh / hin;
        const int32_t y = static_cast<int32_t>(nh - n * hin);
        const int32_t is = __ldg(rh.start + y), ie = __ldg(rh.end + y);
        const int32_t js = __ldg(rw.start + x), je = __ldg(rw.end + x);
        float acc[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            acc[k] = 0.0f;
        }
        for (int32_t i = is; i < ie; ++i) {
            const int32_t loY = __ldg(th.lo + i), hiY = __ldg(th.hi + i);
            const float dY = __ldg(th.delta + i);
            for (int32_t j = js; j < je; ++j) {
                const int32_t loX = __ldg(tw.lo + j), hiX = __ldg(tw.hi + j);
                const float dX = __ldg(tw.delta + j);
                float v[V];
                LoadPackLdg<TIn, V>(go + ((n * hout + i) * wout + j) * static_cast<int64_t>(c) + g * V, v);
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    acc[k] = GatherTap(acc[k], v[k], y, x, loY, hiY, dY, loX, hiX, dX);
                }
            }
        }
        StorePack<TOut, V>(gi + pix * c + static_cast<int64_t>(g) * V, acc);
    }
}

// ---- backward, atomic ---------------------------------------------------------------------------------------
template <typename TIn, int V, int LAY>
__global__ void __launch_bounds__(kThreads)
    BilinearBwdAtomicKernel(const TIn* __restrict__ go, float* __restrict__ acc, int32_t c, int32_t hin, int32_t win,
                            int32_t hout, int32_t wout, LerpAxis th, LerpAxis tw, int64_t totalGroups)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; gid < totalGroups; gid += stride) {
        float v[V];
        LoadPackLdg<TIn, V>(go + gid * V, v);
        if constexpr (LAY == kNCHW) {
            const int32_t groups = wout / V;
            const int64_t row = gid / groups;
            const int32_t g = static_cast<int32_t>(gid - row * groups);
            const int64_t p = row / hout;
            const int32_t h = static_cast<int32_t>(row - p * hout);
            const int32_t loY = __ldg(th.lo + h), hiY = __ldg(th.hi + h);
            const float dY = __ldg(th.delta + h), dY1 = Sub(1.0f, dY);
            float* ap = acc + p * hin * static_cast<int64_t>(win);
#pragma unroll
            for (int k = 0; k < V; ++k) {
                const int32_t w = g * V + k;
                const int32_t loX = __ldg(tw.lo + w), hiX = __ldg(tw.hi + w);
                const float dX = __ldg(tw.delta + w), dX1 = Sub(1.0f, dX);
                atomicAdd(ap + static_cast<int64_t>(loY) * win + loX, Mul(Mul(dX1, dY1), v[k]));
                atomicAdd(ap + static_cast<int64_t>(loY) * win + hiX, Mul(Mul(dX, dY1), v[k]));
                atomicAdd(ap + static_cast<int64_t>(hiY) * win + loX, Mul(Mul(dX1, dY), v[k]));
                atomicAdd(ap + static_cast<int64_t>(hiY) * win + hiX, Mul(Mul(dX, dY), v[k]));
            }
        } else {
            const int32_t groups = c / V;
            const int64_t pix = gid / groups;
            const int32_t g = static_cast<int32_t>(gid - pix * groups);
            const int64_t nh = pix / wout;
            const int32_t w = static_cast<int32_t>(pix - nh * wout);
            const int64_t n = nh / hout;
            const int32_t h = static_cast<int32_t>(nh - n * hout);
            const int32_t loY = __ldg(th.lo + h), hiY = __ldg(th.hi + h);
            const int32_t loX = __ldg(tw.lo + w), hiX = __ldg(tw.hi + w);
            const float dY = __ldg(th.delta + h), dY1 = Sub(1.0f, dY);
            const float dX = __ldg(tw.delta + w), dX1 = Sub(1.0f, dX);
            float* an = acc + n * hin * static_cast<int64_t>(win) * c + g * V;
#pragma unroll
            for (int k = 0; k < V; ++k) {
                atomicAdd(an + (static_cast<int64_t>(loY) * win + loX) * c + k, Mul(Mul(dX1, dY1), v[k]));
                atomicAdd(an + (static_cast<int64_t>(loY) * win + hiX) * c + k, Mul(Mul(dX, dY1), v[k]));
                atomicAdd(an + (static_cast<int64_t>(hiY) * win + loX) * c + k, Mul(Mul(dX1, dY), v[k]));
                atomicAdd(an + (static_cast<int64_t>(hiY) * win + hiX) * c + k, Mul(Mul(dX, dY), v[k]));
            }
        }
    }
}


// Significant bits of a weight (0 for zero). A weight of b bits times a 16-bit value of m significand bits is exact in
// fp32 when b + m <= 24; a fused multiply-add then gives the same bits as the reference's multiply, multiply, add.
int SignificantBits(float w)
{
    uint32_t u;
    std::memcpy(&u, &w, sizeof(u));
    if ((u & 0x7fffffffu) == 0) {
        return 0;
    }
    if (((u >> 23) & 0xffu) == 0) {
        return 24; // subnormal: not worth reasoning about
    }
    uint32_t m = (u & 0x7fffffu) | 0x800000u;
    int bits = 24;
    while ((m & 1u) == 0) {
        m >>= 1;
        --bits;
    }
    return bits;
}

bool IsW2ForwardPattern(const host::Lerp& t, int32_t in)
{
    const int32_t out = static_cast<int32_t>(t.lo.size());
    if (out != 2 * in) {
        return false;
    }
    for (int32_t w = 0; w < out; ++w) {
        const int32_t lo = std::max((w - 1) >> 1, 0), hi = w ? std::min((w + 1) >> 1, in - 1) : 0;
        if (t.lo[w] != lo || t.hi[w] != hi) {
            return false;
        }
    }
    return true;
}

bool IsW2BackwardPattern(const host::Ranges& r, int32_t in, int32_t out)
{
    if (out != 2 * in) {
        return false;
    }
    for (int32_t x = 0; x < in; ++x) {
        const int32_t start = std::max(2 * x - 1, 0), end = std::min(2 * x + 3, out);
        const bool startOk = r.start[x] == start || (x == 1 && r.start[x] == 0);
        if (!startOk || r.end[x] != end) {
            return false;
        }
    }
    return true;
}

// Block shape (column threads, planes per block).
dim3 PlaneBlock(int32_t groups, int64_t planes, int32_t maxPlanes = 256, int32_t maxThreads = kThreads)
{
    const int32_t ct = std::max(1, std::min(groups, maxThreads));
    int64_t pb = std::max(1, maxThreads / ct);
    pb = std::min<int64_t>({pb, planes, static_cast<int64_t>(maxPlanes)});
    return dim3(static_cast<unsigned>(ct), static_cast<unsigned>(std::max<int64_t>(pb, 1)), 1);
}

// Rows per block for the kernels that do not stage: whole planes when there are many, bands when there are few.
int32_t RowsForOccupancy(int64_t threadsPerTileRowSet, int32_t rows)
{
    // enough tiles for about two full waves of resident threads, but walks of at least 8 rows
    const int64_t wantThreads = static_cast<int64_t>(NumSMs()) * 2048 * 2;
    if (threadsPerTileRowSet >= wantThreads) {
        return rows;
    }
    const int64_t tiles = CeilDiv(wantThreads, threadsPerTileRowSet > 0 ? threadsPerTileRowSet : 1);
    return static_cast<int32_t>(std::max<int64_t>({8, CeilDiv(rows, tiles), CeilDiv(rows, 65535)}));
}

template <typename TIn, typename TOut>
cudaError_t LaunchGather(Layout lay, const void* go, void* gi, Shape4 sh, LerpAxis th, LerpAxis tw, RangeAxis rh,
                         RangeAxis rw, const BilinearPlan& plan, cudaStream_t s, bool buildTables,
                         const ViewStrides* gradsPitch)
{
    const int64_t planes = sh.n * sh.c;
    ViewStrides gp; // grad_output dense unless the caller passes a view (only with BilinearBwdTakesPitch)
    gp.n = sh.c * static_cast<int64_t>(sh.hout) * sh.wout;
    gp.c = static_cast<int64_t>(sh.hout) * sh.wout;
    gp.h = sh.wout;
    gp.w = 1;
    gp.chan = static_cast<int32_t>(sh.c);
    if (gradsPitch != nullptr) {
        gp = *gradsPitch;
    }
    // buildTables: the tables and ranges are workspace that has not been filled; they are built here (from the
    // geometry in the plan) unless the kernel chosen below evaluates the entries it needs itself
    bool tablesBuilt = !buildTables;
    cudaError_t tableError = cudaSuccess;
    auto needTables = [&]() {
        if (!tablesBuilt) {
            tableError = BuildLerpBwdTablesAndRanges(plan.geomH, plan.geomW, plan.halfPixel, th, tw, rh, rw, s);
            tablesBuilt = true;
        }
    };
    if (lay == kNCHW) {
        const int v = PickVec(sizeof(TOut), sh.win, {gi});
        const TIn* pg = static_cast<const TIn*>(go);
        TOut* po = static_cast<TOut*>(gi);
        const bool w2 = plan.schedule == BilinearPlan::kW2 || plan.schedule == BilinearPlan::kX2;
        if (w2 && v >= 4 && Aligned(go, 16)) {
            int32_t tileRows = RowsForOccupancy(planes * (sh.win / 4), sh.hin);
            if (plan.schedule == BilinearPlan::kX2) {
                // every tile reduces three extra grads rows before its first output: taller tiles measured faster
                // (28 rows: 81 us, 10 rows: 92 us on fp16 32x256x112x112 -> 56x56) as long as a wave stays full
                tileRows = std::max(tileRows, std::min(sh.hin, 28));
            }
            const int32_t tiles = static_cast<int32_t>(CeilDiv(sh.hin, tileRows));
            const bool x2 = plan.schedule == BilinearPlan::kX2;
            // kX2 with periodic weights and 16-bit tensors: eight grad_input columns per thread
            const bool x2Wide = x2 && plan.periodicW && sizeof(TIn) == 2 && sizeof(TOut) == 2 && sh.win % 8 == 0 &&
                                Aligned(gi, 16);
            const int32_t x2Cols = x2Wide ? 8 : 4;
            const dim3 block = PlaneBlock(sh.win / x2Cols, planes, 256, x2 ? kW2Threads : kThreads);
            const dim3 grid(static_cast<unsigned>(CeilDiv(planes, block.y)), static_cast<unsigned>(tiles));
            // kX2: one wave of resident blocks shares the rows of all plane groups equally
            const int32_t x2Threads = static_cast<int32_t>(block.x * block.y);
            const int64_t x2Total = CeilDiv(planes, block.y) * sh.hin;
            cudaError_t attr = cudaSuccess;
            auto launchX2 = [&](auto kernel) {
                int perSm = 0;
                int32_t rows = 0;
                unsigned blocks = 0;
                size_t bytes = 0;
                // tile height first for a full machine at five blocks per SM, then for what really fits
                for (int pass = 0; pass < 2 && attr == cudaSuccess; ++pass) {
                    const int64_t slots = static_cast<int64_t>(NumSMs()) * (pass == 0 ? 5 : std::max(perSm, 1));
                    const int64_t nb = std::max<int64_t>(1, std::min(slots, x2Total / 8));
                    blocks = static_cast<unsigned>(nb);
                    rows = static_cast<int32_t>(std::min<int64_t>(sh.hin, CeilDiv(x2Total, nb)));
                    bytes = X2SmemBytes(rows, x2Threads, sizeof(TIn), x2Cols);
                    if (bytes > 100 * 1024) {
                        attr = cudaErrorInvalidValue;
                        break;
                    }
                    if (bytes > 48 * 1024) {
                        attr = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                    static_cast<int>(bytes));
                    }
                    if (attr == cudaSuccess) {
                        attr = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, kernel, x2Threads, bytes);
                    }
                    if (attr == cudaSuccess && perSm < 1) {
                        attr = cudaErrorInvalidValue;
                    }
                }
                (void)cudaGetLastError();
                if (attr == cudaSuccess) {
                    kernel<<<blocks, block, bytes, s>>>(pg, po, planes, sh.hin, sh.win, th, tw, rh, rows, plan.bw[0],
                                                        plan.bw[1], plan.bw[2], plan.bw[3], plan.geomH, plan.geomW,
                                                        plan.halfPixel ? 1 : 0, plan.rowStart1, gp);
                }
            };
            if (!(x2 && plan.periodicW)) {
                needTables(); // the periodic variants evaluate their own entries
            }
            if (x2) {
                if (x2Wide) {
                    if constexpr (sizeof(TIn) == 2 && sizeof(TOut) == 2) {
                        if (gradsPitch != nullptr) {
                            launchX2(BilinearBwdX2Kernel<TIn, TOut, false, 8, true, true>);
                        } else {
                            launchX2(BilinearBwdX2Kernel<TIn, TOut, false, 8, true, false>);
                        }
                    }
                } else if (plan.periodicW) {
                    if (gradsPitch != nullptr) {
                            launchX2(BilinearBwdX2Kernel<TIn, TOut, false, 4, true, true>);
                        } else {
                            launchX2(BilinearBwdX2Kernel<TIn, TOut, false, 4, true, false>);
                        }
                } else if (plan.zeroTwins) {
                    if (gradsPitch != nullptr) {
                            launchX2(BilinearBwdX2Kernel<TIn, TOut, true, 4, false, true>);
                        } else {
                            launchX2(BilinearBwdX2Kernel<TIn, TOut, true, 4, false, false>);
                        }
                } else {
                    if (gradsPitch != nullptr) {
                            launchX2(BilinearBwdX2Kernel<TIn, TOut, false, 4, false, true>);
                        } else {
                            launchX2(BilinearBwdX2Kernel<TIn, TOut, false, 4, false, false>);
                        }
                }
            }
            if (x2 && attr == cudaSuccess) {
                // launched above
            } else {
                needTables(); // also after a periodic variant that could not be launched
                BilinearBwdW2Kernel<TIn, TOut><<<grid, block, 0, s>>>(pg, po, planes, sh.hin, sh.win, sh.hout, th, tw,
                                                                      rh, tileRows);
            }
        } else if (plan.schedule != BilinearPlan::kDirect && plan.tileRows > 0) {
            needTables();
            const int32_t tiles = static_cast<int32_t>(CeilDiv(sh.hin, plan.tileRows));
            const int32_t stride = static_cast<int32_t>(
                (StageBytes(static_cast<int64_t>(plan.bandRows) * sh.wout, sizeof(TIn)) + 15) & ~size_t(15));
            const int vv = std::min(v, 4);
            OPSCV_DISPATCH_VEC(vv, V, {
                if constexpr (V <= 4) {
                    const dim3 block = PlaneBlock(sh.win / V, planes, plan.planesPerBlock);
                    const dim3 grid(static_cast<unsigned>(CeilDiv(planes, block.y)), static_cast<unsigned>(tiles));
                    const size_t smem = static_cast<size_t>(stride) * block.y;
                    if (plan.tapsW <= 4) {
                        BilinearBwdTileKernel<TIn, TOut, V, 4><<<grid, block, smem, s>>>(
                            pg, po, planes, sh.hin, sh.win, sh.hout, sh.wout, th, tw, rh, rw, plan.tileRows, stride);
                    } else {
                        BilinearBwdTileKernel<TIn, TOut, V, 8><<<grid, block, smem, s>>>(
                            pg, po, planes, sh.hin, sh.win, sh.hout, sh.wout, th, tw, rh, rw, plan.tileRows, stride);
                    }
                }
            });
        } else {
            needTables();
            OPSCV_DISPATCH_VEC(v, V, {
                if constexpr (V * sizeof(TOut) <= 16) {
                    const int64_t total = planes * sh.hin * (sh.win / V);
                    BilinearBwdGatherNCHWKernel<TIn, TOut, V><<<GridFor(total, kThreads), kThreads, 0, s>>>(
                        pg, po, sh.hin, sh.win, sh.hout, sh.wout, th, tw, rh, rw, total);
                }
            });
        }
    } else {
        needTables();
        const int elem = sizeof(TIn) > sizeof(TOut) ? sizeof(TIn) : sizeof(TOut);
        const int v = PickVec(elem, sh.c, {go, gi});
        OPSCV_DISPATCH_VEC(v, V, {
            if constexpr (V * sizeof(TIn) <= 16 && V * sizeof(TOut) <= 16) {
                const int64_t total = sh.n * sh.hin * sh.win * (sh.c / V);
                BilinearBwdGatherNHWCKernel<TIn, TOut, V><<<GridFor(total, kThreads), kThreads, 0, s>>>(
                    static_cast<const TIn*>(go), static_cast<TOut*>(gi), static_cast<int32_t>(sh.c), sh.hin, sh.win,
                    sh.hout, sh.wout, th, tw, rh, rw, total);
            }
        });
    }
    CountLaunch();
    if (tableError != cudaSuccess) {
        return tableError;
    }
    return cudaGetLastError();
}

} // namespace

BilinearPlan MakeBilinearFwdPlan(Dt dt, Layout lay, Shape4 sh, AxisGeom gh, AxisGeom gw, bool halfPixel)
{
    BilinearPlan plan{};
    plan.schedule = BilinearPlan::kDirect;
    plan.geomH = gh;
    plan.geomW = gw;
    plan.halfPixel = halfPixel;
    if (lay != kNCHW) {
        if (DtSize(dt) == 2) { // can the 16-bit walker fuse its horizontal interpolation?
            const host::Lerp tW = host::LerpTable(sh.win, sh.wout, gw.scale, halfPixel, 0);
            int bits = 0;
            for (float d : tW.delta) {
                bits = std::max({bits, SignificantBits(d), SignificantBits(1.0f - d)});
            }
            plan.weightSlack = 24 - bits;
        }
        if (sh.hout == 2 * sh.hin) {
            const host::Lerp tH = host::LerpTable(sh.hin, sh.hout, gh.scale, halfPixel, 0);
            bool x2 = tH.lo[0] == 0 && tH.hi[0] == 0 && tH.lo[sh.hout - 1] == sh.hin - 1 && tH.hi[sh.hout - 1] == sh.hin - 1;
            for (int32_t i = 0; i + 1 < sh.hin && x2; ++i) {
                x2 = tH.lo[2 * i + 1] == i && tH.hi[2 * i + 1] == i + 1 && tH.lo[2 * i + 2] == i && tH.hi[2 * i + 2] == i + 1;
            }
            plan.rowsX2 = x2;
        }
        return plan;
    }
    const int es = DtSize(dt);
    const host::Lerp tH = host::LerpTable(sh.hin, sh.hout, gh.scale, halfPixel, 0);
    const host::Lerp tW = host::LerpTable(sh.win, sh.wout, gw.scale, halfPixel, 0);
    if (sh.win % 4 == 0 && IsW2ForwardPattern(tW, sh.win)) {
        plan.schedule = BilinearPlan::kW2;
        plan.periodicW = true;
        for (int32_t w = 3; w < sh.wout; ++w) {
            plan.periodicW = plan.periodicW && std::memcmp(&tW.delta[w], &tW.delta[w - 2], sizeof(float)) == 0;
        }
        plan.dxFirst = tW.delta[0];
        plan.dxEven = tW.delta[2];
        plan.dxOdd = tW.delta[1];
        int bits = 0;
        for (float w : {plan.dxFirst, plan.dxEven, plan.dxOdd}) {
            bits = std::max({bits, SignificantBits(w), SignificantBits(1.0f - w)});
        }
        plan.weightSlack = 24 - bits;
        if (sh.hout == 2 * sh.hin) {
            bool x2 = tH.lo[0] == 0 && tH.hi[0] == 0 && tH.lo[sh.hout - 1] == sh.hin - 1 && tH.hi[sh.hout - 1] == sh.hin - 1;
            for (int32_t i = 0; i + 1 < sh.hin && x2; ++i) {
                x2 = tH.lo[2 * i + 1] == i && tH.hi[2 * i + 1] == i + 1 && tH.lo[2 * i + 2] == i && tH.hi[2 * i + 2] == i + 1;
            }
            plan.rowsX2 = x2;
        }
        return plan;
    }
    // Several planes share a block (uniform row walks, full warps even for narrow images); their bands share the
    // staging budget. Aim for bands of at least 8 input rows, with fewer planes per block if rows are long.
    const int64_t rowBytes = static_cast<int64_t>(sh.win) * es;
    const int32_t vMax = std::min(4, 16 / es);
    int32_t pb = static_cast<int32_t>(PlaneBlock(std::max(1, sh.wout / vMax), sh.n * sh.c).y);
    pb = static_cast<int32_t>(std::max<int64_t>(1, std::min<int64_t>(pb, kStageBudget / (rowBytes * 8 + 32))));
    const int32_t budgetRows = static_cast<int32_t>(std::min<int64_t>((kStageBudget / pb - 32) / rowBytes, sh.hin));
    auto need = [&](int32_t h0, int32_t h1) { return tH.hi[h1 - 1] - tH.lo[h0] + 1; };
    int32_t tileRows = host::PickTileRows(sh.hout, budgetRows, need);
    if (tileRows > 0) { // no taller than needed to keep the machine busy
        tileRows = std::min(tileRows, RowsForOccupancy(sh.n * sh.c * std::max(1, sh.wout / vMax), sh.hout));
    }
    if (tileRows > 0 && sh.n * sh.c < (1LL << 31) && CeilDiv(sh.hout, tileRows) <= 65535) {
        plan.schedule = BilinearPlan::kTiled;
        plan.tileRows = tileRows;
        plan.bandRows = host::MaxBand(sh.hout, tileRows, need);
        plan.planesPerBlock = pb;
    }
    return plan;
}

BilinearPlan MakeBilinearBwdPlan(Dt dtIn, Layout lay, Shape4 sh, AxisGeom gh, AxisGeom gw, bool halfPixel)
{
    BilinearPlan plan{};
    plan.schedule = BilinearPlan::kDirect;
    plan.geomH = gh;
    plan.geomW = gw;
    plan.halfPixel = halfPixel;
    if (lay != kNCHW) {
        return plan;
    }
    const int es = DtSize(dtIn);
    const host::Lerp tH = host::LerpTable(sh.hin, sh.hout, gh.scale, halfPixel, 1);
    const host::Lerp tW = host::LerpTable(sh.win, sh.wout, gw.scale, halfPixel, 1);
    const host::Ranges rH = host::LerpBwdRanges(tH, sh.hin);
    const host::Ranges rW = host::LerpBwdRanges(tW, sh.win);
    // clamped-border sources whose two taps share an index and one weight is exactly zero (align_corners)
    auto hasTwins = [](const host::Lerp& t) {
        for (size_t j = 0; j < t.lo.size(); ++j) {
            if (t.lo[j] == t.hi[j] && (t.delta[j] == 0.0f || t.delta[j] == 1.0f)) {
                return true;
            }
        }
        return false;
    };
    plan.zeroTwins = hasTwins(tH) || hasTwins(tW);
    if (sh.win % 4 == 0 && IsW2BackwardPattern(rW, sh.win, sh.wout)) {
        plan.schedule = IsW2BackwardPattern(rH, sh.hin, sh.hout) ? BilinearPlan::kX2 : BilinearPlan::kW2;
        // weight of grads column j for grad_input column x, as the kernels combine it
        auto combined = [&](int32_t j, int32_t x) {
            float w = 0.0f;
            if (tW.lo[j] == x) {
                w = 1.0f - tW.delta[j];
            }
            if (tW.hi[j] == x) {
                w = w + tW.delta[j];
            }
            return w;
        };
        plan.rowStart1 = sh.hin > 1 ? rH.start[1] : 0;
        plan.periodicW = plan.schedule == BilinearPlan::kX2 && !plan.zeroTwins && sh.win >= 3;
        if (plan.periodicW) {
            for (int t = 0; t < 4; ++t) {
                plan.bw[t] = combined(1 + t, 1);
            }
            for (int32_t x = 1; x + 1 < sh.win && plan.periodicW; ++x) {
                for (int t = 0; t < 4; ++t) {
                    const float w = combined(2 * x - 1 + t, x);
                    plan.periodicW = plan.periodicW && std::memcmp(&w, &plan.bw[t], sizeof(float)) == 0;
                }
            }
        }
        return plan;
    }
    int32_t taps = 0;
    for (int32_t x = 0; x < sh.win; ++x) {
        taps = std::max(taps, rW.end[x] - rW.start[x]);
    }
    const int64_t rowBytes = static_cast<int64_t>(sh.wout) * es;
    const int32_t vMax = std::min(4, 16 / es);
    int32_t pb = static_cast<int32_t>(PlaneBlock(std::max(1, sh.win / vMax), sh.n * sh.c).y);
    pb = static_cast<int32_t>(std::max<int64_t>(1, std::min<int64_t>(pb, kStageBudget / (rowBytes * 8 + 32))));
    const int32_t budgetRows = static_cast<int32_t>(std::min<int64_t>((kStageBudget / pb - 32) / rowBytes, sh.hout));
    auto need = [&](int32_t y0, int32_t y1) { return std::max(0, rH.end[y1 - 1] - rH.start[y0]); };
    int32_t tileRows = taps <= 8 ? host::PickTileRows(sh.hin, budgetRows, need) : 0;
    if (tileRows > 0) {
        tileRows = std::min(tileRows, RowsForOccupancy(sh.n * sh.c * std::max(1, sh.win / vMax), sh.hin));
    }
    if (tileRows > 0 && sh.n * sh.c < (1LL << 31) && CeilDiv(sh.hin, tileRows) <= 65535) {
        plan.schedule = BilinearPlan::kTiled;
        plan.tileRows = tileRows;
        plan.bandRows = host::MaxBand(sh.hin, tileRows, need);
        plan.tapsW = taps;
        plan.planesPerBlock = pb;
    }
    return plan;
}

bool BilinearFwdTakesPitch(Dt dt, Layout lay, const void* x, const void* y, Shape4 sh, const BilinearPlan& plan,
                           const ViewStrides& in, const ViewStrides& out)
{
    const size_t es = static_cast<size_t>(DtSize(dt));
    // the conditions of the 2x-width kernel below, with the views' pitches in place of the dense ones (the input
    // queue copies 16 bytes at a time)
    return lay == kNCHW && plan.schedule == BilinearPlan::kW2 && out.w == 1 && in.w == 1 && Aligned(x, 16) &&
           Aligned(y, 16) && (sh.wout * es) % 16 == 0 && (out.n * es) % 16 == 0 && (out.c * es) % 16 == 0 &&
           (out.h * es) % 16 == 0 && (in.n * es) % 16 == 0 && (in.c * es) % 16 == 0 && (in.h * es) % 16 == 0;
}

cudaError_t BilinearFwd(Dt dt, Layout lay, const void* x, void* y, Shape4 sh, LerpAxis th, LerpAxis tw,
                        const BilinearPlan& plan, cudaStream_t s, bool buildTables, const ViewStrides* outPitch,
                        const ViewStrides* inPitch)
{
    const int64_t planes = sh.n * sh.c;
    ViewStrides ip; // dense input unless the caller passes a view
    ip.n = sh.c * static_cast<int64_t>(sh.hin) * sh.win;
    ip.c = static_cast<int64_t>(sh.hin) * sh.win;
    ip.h = sh.win;
    ip.w = 1;
    ip.chan = static_cast<int32_t>(sh.c);
    if (inPitch != nullptr) {
        ip = *inPitch;
    }
    ViewStrides op; // dense output unless the caller passes a view (only with BilinearFwdTakesPitch)
    op.n = sh.c * static_cast<int64_t>(sh.hout) * sh.wout;
    op.c = static_cast<int64_t>(sh.hout) * sh.wout;
    op.h = sh.wout;
    op.w = 1;
    op.chan = static_cast<int32_t>(sh.c);
    if (outPitch != nullptr) {
        op = *outPitch;
    }
    // buildTables: th / tw are still empty; they are filled here (from the geometry in the plan) unless the kernel
    // chosen below evaluates the entries it needs itself
    bool tablesBuilt = !buildTables;
    cudaError_t tableError = cudaSuccess;
    auto needTables = [&]() {
        if (!tablesBuilt) {
            tableError = BuildLerpTables(plan.geomH, plan.geomW, plan.halfPixel, 0, th, tw, s);
            tablesBuilt = true;
        }
    };
    OPSCV_DISPATCH_DT(dt, T, {
        if (lay == kNCHW) {
            const int v = PickVec(sizeof(T), sh.wout, {y});
            const T* px = static_cast<const T*>(x);
            T* py = static_cast<T*>(y);
            // the 2x kernel loads 4 input columns and stores 8 output columns per thread as vectors
            const bool w2Ok = plan.schedule == BilinearPlan::kW2 && Aligned(x, 4 * sizeof(T)) &&
                              Aligned(y, sizeof(T) == 2 ? 16 : 16) && (sh.wout * sizeof(T)) % 16 == 0;
            if (!w2Ok) {
                needTables();
            }
            if (w2Ok) {
                // 16-bit tensors: eight input columns (one 16-byte load) per thread when the rows allow it
                const int vi = (sizeof(T) == 2 && sh.win % 8 == 0 && Aligned(x, 16)) ? 8 : 4;
                // one wave of resident blocks shares the output rows of all plane groups equally; runs of at
                // least 8 rows
                const int32_t tileRows = std::min(sh.hout, 512);
                const dim3 block = PlaneBlock(sh.win / vi, planes, 256, kW2Threads);
                const int64_t totalRows = CeilDiv(planes, block.y) * sh.hout;
                // a thread writes 2 * vi elements per row; when that is 32 bytes and the rows are 32-byte aligned
                // they go out as one 32-byte store
                const int32_t wide = (2 * vi * sizeof(T) == 32 && Aligned(y, 32) && (sh.wout * sizeof(T)) % 32 == 0 &&
                                      (op.n * sizeof(T)) % 32 == 0 && (op.c * sizeof(T)) % 32 == 0 &&
                                      (op.h * sizeof(T)) % 32 == 0) ? 1 : 0;
                // 16-byte pieces (fp32 x 4, 16-bit x 8) stream through the per-thread queue
                const size_t qBytes = static_cast<size_t>(kW2QueueDepth) * block.x * block.y * 24;
                auto launch = [&](auto kernel, size_t smem, bool periodic) {
                    if (periodic) {
                        smem += static_cast<size_t>(tileRows) * 16; // the tile's row entries
                    } else {
                        needTables();
                    }
                    int perSm = 0;
                    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, kernel, static_cast<int>(block.x * block.y),
                                                                      smem) != cudaSuccess || perSm < 1) {
                        (void)cudaGetLastError();
                        perSm = 1;
                    }
                    const dim3 grid(static_cast<unsigned>(std::max<int64_t>(
                        1, std::min<int64_t>(static_cast<int64_t>(NumSMs()) * perSm, totalRows / 8))));
                    kernel<<<grid, block, smem, s>>>(px, py, planes, sh.hin, sh.win, sh.hout, th, tw, tileRows, wide,
                                                     plan.dxFirst, plan.dxEven, plan.dxOdd, plan.geomH,
                                                     plan.halfPixel ? 1 : 0, op, ip);
                };
                if (vi == 8) {
                    if constexpr (sizeof(T) == 2) {
                        // significand bits of T: 11 (fp16), 8 (bf16)
                        const int mant = std::is_same<T, __half>::value ? 11 : 8;
                        if (plan.periodicW && mant <= plan.weightSlack) {
                            if (outPitch != nullptr) {
                            launch(BilinearFwdW2Kernel<T, 8, true, true, true, true>, qBytes, true);
                        } else {
                            if (plan.rowsX2) { // 56.2 us against 56.8 us at the FPN shapes
                                launch(BilinearFwdW2Kernel<T, 8, true, true, true, false, true>, qBytes, true);
                            } else {
                                launch(BilinearFwdW2Kernel<T, 8, true, true, true, false>, qBytes, true);
                            }
                        }
                        } else if (plan.periodicW) {
                            if (outPitch != nullptr) {
                            launch(BilinearFwdW2Kernel<T, 8, true, true, false, true>, qBytes, true);
                        } else {
                            launch(BilinearFwdW2Kernel<T, 8, true, true, false, false>, qBytes, true);
                        }
                        } else {
                            if (outPitch != nullptr) {
                            launch(BilinearFwdW2Kernel<T, 8, true, false, false, true>, qBytes, false);
                        } else {
                            launch(BilinearFwdW2Kernel<T, 8, true, false, false, false>, qBytes, false);
                        }
                        }
                    }
                } else if (sizeof(T) == 4) {
                    if constexpr (sizeof(T) == 4) {
                        if (plan.periodicW) {
                            if (outPitch != nullptr) {
                            launch(BilinearFwdW2Kernel<T, 4, true, true, false, true>, qBytes, true);
                        } else {
                            launch(BilinearFwdW2Kernel<T, 4, true, true, false, false>, qBytes, true);
                        }
                        } else {
                            if (outPitch != nullptr) {
                            launch(BilinearFwdW2Kernel<T, 4, true, false, false, true>, qBytes, false);
                        } else {
                            launch(BilinearFwdW2Kernel<T, 4, true, false, false, false>, qBytes, false);
                        }
                        }
                    }
                } else {
                    if (outPitch != nullptr) {
                            launch(BilinearFwdW2Kernel<T, 4, false, false, false, true>, 0, false);
                        } else {
                            launch(BilinearFwdW2Kernel<T, 4, false, false, false, false>, 0, false);
                        }
                }
            } else if (plan.schedule == BilinearPlan::kTiled && plan.tileRows > 0) {
                const int32_t tiles = static_cast<int32_t>(CeilDiv(sh.hout, plan.tileRows));
                const int32_t stride = static_cast<int32_t>(
                    (StageBytes(static_cast<int64_t>(plan.bandRows) * sh.win, sizeof(T)) + 15) & ~size_t(15));
                const int vv = std::min(v, 4);
                OPSCV_DISPATCH_VEC(vv, V, {
                    if constexpr (V <= 4) {
                        const dim3 block = PlaneBlock(sh.wout / V, planes, plan.planesPerBlock);
                        const dim3 grid(static_cast<unsigned>(CeilDiv(planes, block.y)), static_cast<unsigned>(tiles));
                        BilinearFwdTileKernel<T, V><<<grid, block, static_cast<size_t>(stride) * block.y, s>>>(
                            px, py, planes, sh.hin, sh.win, sh.hout, sh.wout, th, tw, plan.tileRows, stride);
                    }
                });
            } else {
                OPSCV_DISPATCH_VEC(v, V, {
                    if constexpr (V * sizeof(T) <= 16) {
                        // Split the rows of a plane into chunks only as far as needed to fill the machine (longer
                        // walks reuse more rows).
                        const int64_t columns = planes * (sh.wout / V);
                        const int64_t wanted = static_cast<int64_t>(NumSMs()) * 2048 * 2;
                        int64_t chunks = CeilDiv(wanted, columns > 0 ? columns : 1);
                        chunks = chunks < 1 ? 1 : (chunks > sh.hout ? sh.hout : chunks);
                        const int32_t rows = static_cast<int32_t>(CeilDiv(sh.hout, chunks));
                        const int32_t rowChunks = static_cast<int32_t>(CeilDiv(sh.hout, rows));
                        const int64_t total = columns * rowChunks;
                        BilinearFwdNCHWKernel<T, V><<<GridFor(total, kThreads, 16), kThreads, 0, s>>>(
                            px, py, sh.hin, sh.win, sh.hout, sh.wout, th, tw, rows, rowChunks, total);
                    }
                });
            }
        } else {
            needTables();
            const int v = PickVec(sizeof(T), sh.c, {x, y});
            OPSCV_DISPATCH_VEC(v, V, {
                if constexpr (V * sizeof(T) <= 16) {
                    // One walker per (image, output column, channel vector); the rows are cut into chunks only
                    // as far as needed to give every SM a few thousand threads.
                    const int64_t walkers = sh.n * sh.wout * (sh.c / V);
                    const int64_t wanted = static_cast<int64_t>(NumSMs()) * 2048 * 2;
                    int64_t chunks = CeilDiv(wanted, walkers > 0 ? walkers : 1);
                    chunks = std::max<int64_t>(1, std::min<int64_t>(chunks, CeilDiv(sh.hout, 4)));
                    const int32_t rows = static_cast<int32_t>(CeilDiv(sh.hout, chunks));
                    const int32_t rowChunks = static_cast<int32_t>(CeilDiv(sh.hout, rows));
                    const unsigned blocks = static_cast<unsigned>(
                        std::min<int64_t>(CeilDiv(walkers * rowChunks, kThreads), 0x7fffffff));
                    bool queued = false;
                    if constexpr (V * sizeof(T) == 16) {
                        if (Aligned(x, 16)) {
                            const size_t qBytes = static_cast<size_t>(kFwdQueueDepth) * kThreads * 32;
                            const int mant = std::is_same<T, __half>::value ? 11 : 8; // significand bits of T
                            const bool x2Rows = plan.rowsX2 && sh.hout == 2 * sh.hin;
                            // the 2x walk is cut into chunks of steps (one new input row each) instead of output rows
                            const int32_t steps = std::max(sh.hin - 1, 1);
                            const int32_t stepRows = static_cast<int32_t>(CeilDiv(steps, std::min<int64_t>(chunks, steps)));
                            const int32_t stepChunks = static_cast<int32_t>(CeilDiv(steps, stepRows));
                            auto launch = [&](auto kernel, bool stepped) {
                                const int32_t r = stepped ? stepRows : rows, rc = stepped ? stepChunks : rowChunks;
                                const unsigned nb = static_cast<unsigned>(std::min<int64_t>(CeilDiv(walkers * rc, kThreads), 0x7fffffff));
                                kernel<<<nb, kThreads, qBytes, s>>>(
                                    static_cast<const T*>(x), static_cast<T*>(y), static_cast<int32_t>(sh.c), sh.hin,
                                    sh.win, sh.hout, sh.wout, th, tw, r, rc, walkers);
                            };
                            if (sizeof(T) == 2 && mant <= plan.weightSlack) {
                                if constexpr (sizeof(T) == 2) {
                                    if (x2Rows) {
                                        launch(BilinearFwdNHWCKernel<T, V, true, true, true>, true);
                                    } else {
                                        launch(BilinearFwdNHWCKernel<T, V, true, true>, false);
                                    }
                                }
                            } else if (x2Rows) {
                                launch(BilinearFwdNHWCKernel<T, V, true, false, true>, true);
                            } else {
                                launch(BilinearFwdNHWCKernel<T, V, true>, false);
                            }
                            queued = true;
                        }
                    }
                    if (!queued) {
    BilinearFwdNHWCKernel<T, V, false><<<blocks, kThreads, 0, s>>>(
                        static_cast<const T*>(x), static_cast<T*>(y), static_cast<int32_t>(sh.c), sh.hin, sh.win,
                        sh.hout, sh.wout, th, tw, rows, rowChunks, walkers);
                    }

                }
            });
        }
    });
    CountLaunch();
    if (tableError != cudaSuccess) {
        return tableError;
    }
    return cudaGetLastError();
}

bool BilinearBwdTakesPitch(Dt dtIn, Dt dtOut, Layout lay, const void* go, const void* gi, Shape4 sh,
                           const BilinearPlan& plan, const ViewStrides& grads)
{
    const size_t es = static_cast<size_t>(DtSize(dtIn));
    // the conditions under which LaunchGather runs the 2x kernel, with the view's pitches in place of the dense ones
    return lay == kNCHW && plan.schedule == BilinearPlan::kX2 && grads.w == 1 &&
           PickVec(DtSize(dtOut), sh.win, {gi}) >= 4 && Aligned(go, 16) && (grads.n * es) % 16 == 0 &&
           (grads.c * es) % 16 == 0 && (grads.h * es) % 16 == 0;
}

cudaError_t BilinearBwdGather(Dt dtIn, Dt dtOut, Layout lay, const void* go, void* gi, Shape4 sh, LerpAxis th,
                              LerpAxis tw, RangeAxis rh, RangeAxis rw, const BilinearPlan& plan, cudaStream_t s,
                              bool buildTables, const ViewStrides* gradsPitch)
{
    if (dtIn == dtOut) {
        OPSCV_DISPATCH_DT(dtIn, T, {
            return (LaunchGather<T, T>(lay, go, gi, sh, th, tw, rh, rw, plan, s, buildTables, gradsPitch));
        });
    }
    if (dtIn == Dt::F32 && dtOut == Dt::F16) {
        return LaunchGather<float, __half>(lay, go, gi, sh, th, tw, rh, rw, plan, s, buildTables, gradsPitch);
    }
    if (dtIn == Dt::F32 && dtOut == Dt::BF16) {
        return LaunchGather<float, __nv_bfloat16>(lay, go, gi, sh, th, tw, rh, rw, plan, s, buildTables, gradsPitch);
    }
    return cudaErrorInvalidValue;
}

cudaError_t BilinearBwdAtomic(Dt dtIn, Dt dtOut, Layout lay, const void* go, void* gi, float* acc, Shape4 sh,
                              LerpAxis th, LerpAxis tw, cudaStream_t s)
{
    const int64_t outElems = sh.n * sh.c * sh.hin * sh.win;
    cudaError_t e = cudaMemsetAsync(acc, 0, static_cast<size_t>(outElems) * sizeof(float), s);
    if (e != cudaSuccess) {
        return e;
    }
    OPSCV_DISPATCH_DT(dtIn, T, {
        const int64_t inner = lay == kNCHW ? sh.wout : sh.c;
        const int v = PickVec(sizeof(T), inner, {go});
        OPSCV_DISPATCH_VEC(v, V, {
            if constexpr (V * sizeof(T) <= 16) {
                const int64_t total = sh.n * sh.c * sh.hout * static_cast<int64_t>(sh.wout) / V;
                if (lay == kNCHW) {
                    BilinearBwdAtomicKernel<T, V, kNCHW><<<GridFor(total, kThreads), kThreads, 0, s>>>(
                        static_cast<const T*>(go), acc, static_cast<int32_t>(sh.c), sh.hin, sh.win, sh.hout, sh.wout,
                        th, tw, total);
                } else {
                    BilinearBwdAtomicKernel<T, V, kNHWC><<<GridFor(total, kThreads), kThreads, 0, s>>>(
                        static_cast<const T*>(go), acc, static_cast<int32_t>(sh.c), sh.hin, sh.win, sh.hout, sh.wout,
                        th, tw, total);
                }
            }
        });
    });
    CountLaunch(2);
    e = cudaGetLastError();
    if (e != cudaSuccess) {
        return e;
    }
    if (dtOut != Dt::F32 || static_cast<void*>(acc) != gi) {
        return CastFromF32(dtOut, gi, acc, outElems, s);
    }
    return cudaSuccess;
}

} // namespace opscv
