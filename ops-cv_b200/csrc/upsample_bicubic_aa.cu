// UpsampleBicubic2dAA forward and backward (NCHW).
//
// The anti-aliased bicubic filter is separable: out[i][j] = sum_m wH[i][m] * sum_n wW[j][n] * x[hmin_i+m][wmin_j+n]
// with per-axis windows and normalised weights that depend only on the output index. tables.cu builds those
// windows / weights once per call; the kernels here never evaluate the cubic.
//
// Forward
//   * streaming kernel (down-scaling, the common case): a block owns a band of output rows of one plane and
//     streams the input rows that band needs exactly once, 16 bytes per thread, fully coalesced. Each thread
//     owns four input columns and carries a small ring of partial sums, one per output row whose vertical window
//     is currently open (an input row touches only ~support/scale output rows). When an output row's window
//     closes, its vertically filtered row (still at input width) goes to shared memory and the block applies the
//     horizontal filter, each thread producing output columns with its weights held in registers.
//     Input is read once from HBM, nothing but the output is written.
//   * direct kernel (any shape): one thread per output element, double loop over the window in the reference's
//     accumulation order (rows outer, columns inner).
// Backward
//   * gather kernel: one thread per grad_input element sums the outputs whose windows cover it, rows outer,
//     columns inner; deterministic. A block-tiled variant serves the down-scaling case, where each output row
//     fans out to many input rows.
//   * atomic kernel: the reference's scatter with fp32 atomics (selectable).
//
// Reference arithmetic: image/upsample_bicubic2d_aa/op_kernel/arch35/upsample_bicubic2d_aa_simt_base.h:52-127,
// image/upsample_bicubic2d_aa_grad/op_kernel/arch35/upsample_bicubic2d_aa_grad_simt_base.h:32-102 and
// upsample_bicubic2d_aa_grad_simt_base_deter.h:30-122.
#include <algorithm>

#include "launch_util.cuh"

namespace opscv {
namespace {

constexpr int kThreads = 256;

// ---- forward, direct ----------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
    AAFwdDirectKernel(const T* __restrict__ x, T* __restrict__ y, int32_t hin, int32_t win, int32_t hout,
                      int32_t wout, AAAxis th, AAAxis tw, int64_t total)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t row = idx / wout;
        const int32_t w = static_cast<int32_t>(idx - row * wout);
        const int64_t p = row / hout;
        const int32_t h = static_cast<int32_t>(row - p * hout);
        const int32_t hmin = __ldg(th.xmin + h), hsz = __ldg(th.xsize + h);
        const int32_t wmin = __ldg(tw.xmin + w), wsz = __ldg(tw.xsize + w);
        const float* wh = th.w + static_cast<int64_t>(h) * th.taps;
        const float* ww = tw.w + static_cast<int64_t>(w) * tw.taps;
        const T* xp = x + p * hin * static_cast<int64_t>(win);
        float value = 0.0f;
        for (int32_t m = 0; m < hsz; ++m) {
            const float weightH = __ldg(wh + m);
            const T* xr = xp + static_cast<int64_t>(hmin + m) * win + wmin;
            for (int32_t n = 0; n < wsz; ++n) {
                // value += x * weightsH * weightsW  (simt_base.h:121)
                value = Add(value, Mul(Mul(DType<T>::Load(xr + n), weightH), __ldg(ww + n)));
            }
        }
        y[idx] = DType<T>::FromF(value);
    }
}

// ---- forward, streaming (down-scaling) -----------------------------------------------------------------------
// Per input row r, the outputs whose vertical window covers r form a short run [start(r), end(r)): for scale >= 1 an
// output covers r iff |centre - (r + 0.5)| < support + 0.5, a span of 4*scale + 1 input pixels that holds at most
// 4 + 1/scale + 1 <= 6 = kSlots centres. AARowWeightKernel tabulates, once per call, the weight of output
// start(r) + a at row r for a < kSlots (0 past the run), followed by start(r) and the run length as integer bit
// patterns: one 32-byte record per input row.
constexpr int kSlots = 6;
constexpr int kSlotStride = 8;
constexpr int kFlushBatch = 4;        // output rows per horizontal pass of the streaming forward kernel
constexpr int kStreamMaxThreads = 256; // up to 255 registers per thread for the accumulator ring and the row queue

__global__ void AARowWeightKernel(AAAxis th, RangeAxis rh, int32_t hin, float* __restrict__ wrow)
{
    const int32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= hin) {
        return;
    }
    const int32_t s = __ldg(rh.start + r), e = __ldg(rh.end + r);
#pragma unroll
    for (int a = 0; a < kSlots; ++a) {
        const int32_t i = s + a;
        float w = 0.0f;
        if (i < e) {
            const int32_t t = r - __ldg(th.xmin + i);
            if (t >= 0 && t < __ldg(th.xsize + i)) {
                w = __ldg(th.w + static_cast<int64_t>(i) * th.taps + t);
            }
        }
        wrow[static_cast<int64_t>(r) * kSlotStride + a] = w;
    }
    // the run itself rides along in the two spare floats of the row, so that one 32-byte read gives everything
    wrow[static_cast<int64_t>(r) * kSlotStride + 6] = __int_as_float(s);
    wrow[static_cast<int64_t>(r) * kSlotStride + 7] = __int_as_float(min(e - s, kSlots));
}

// ---- bulk asynchronous copies (global -> shared) with mbarrier completion ----------------------------------------
// Used by the streaming forward kernel to keep whole input rows in flight without holding them in registers.
// Every wait is bounded: a wait that runs out bumps g_asyncCopyTimeouts (read by AsyncCopyTimeouts()), the block
// waits (bounded again) for the copies it still has in flight and returns, so the context stays usable.
__device__ unsigned int g_asyncCopyTimeouts = 0;
constexpr uint32_t kWaitLimit = 1u << 22;

__device__ __forceinline__ uint32_t SmemAddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void BarrierInit(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void BarrierInitFence()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Arms the barrier for `bytes` of copy traffic and starts one row copy that completes on it. dst, src and bytes are
// multiples of 16.
__device__ __forceinline__ void BulkLoadRow(void* dst, const void* src, uint32_t bytes, uint64_t* bar)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemAddr(bar)), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     SmemAddr(dst)),
                 "l"(src), "r"(bytes), "r"(SmemAddr(bar))
                 : "memory");
}
__device__ __forceinline__ bool BarrierWait(uint64_t* bar, uint32_t parity, uint32_t limit)
{
    const uint32_t addr = SmemAddr(bar);
    for (uint32_t it = 0; it < limit; ++it) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok)
                     : "r"(addr), "r"(parity)
                     : "memory");
        if (ok) {
            return true;
        }
    }
    return false;
}

// The parked rows are skewed by one float per 32 columns: the horizontal pass reads them at a stride of `scale`
// columns per lane, and without the skew lanes 32 / scale apart would always meet in one bank.
__host__ __device__ __forceinline__ int32_t Skew(int32_t col) { return col + (col >> 5); }
__host__ __device__ __forceinline__ int32_t ParkedRowFloats(int32_t win) { return (Skew(win) + 4) & ~3; }

// grid = (planes, bands); a band is `bandRows` output rows. A thread owns VC input columns of every row (one or two
// 16-byte groups) and keeps one partial sum per open output row (kSlots of them) for each.
// Shared memory: the vertically filtered row being flushed, the slot-weight rows of the band's input rows, and
// (wTaps > 0) the horizontal weights of all output columns, transposed.
// Two ways of bringing the input rows in:
//   BULK = false: every thread loads its own columns, PF rows ahead, into registers;
//   BULK = true : thread 0 starts one bulk asynchronous copy per row into a ring of ringGroups * PF row slots in
//                 shared memory (completion on one mbarrier per slot); the rows of a group of PF are consumed by all
//                 threads from shared memory, and after a block barrier the group's slots are refilled with the rows
//                 ringGroups groups ahead. Whole rows are in flight at no register cost.
template <typename T, int VC, int MAXT, bool BULK>
__global__ void __launch_bounds__(MAXT, (VC == 4 && !BULK) ? 4 : (BULK ? 1 : 2))
    AAFwdStreamKernel(const T* __restrict__ x, T* __restrict__ y, int32_t hin, int32_t win, int32_t hout,
                      int32_t wout, AAAxis th, AAAxis tw, const float* __restrict__ wrow, int32_t bandRows,
                      int32_t metaRows, int32_t wTaps, int32_t ringGroups)
{
    // input rows in flight per thread / rows per ring group (two keep the 4-column variant within 64 registers without spills)
    constexpr int PF = (VC == 4 && !BULK) ? 2 : 4;
    constexpr int LV = 16 / sizeof(T);     // elements per 16-byte load
    constexpr int NL = VC / LV;            // 16-byte loads per row
    extern __shared__ __align__(16) float smemAll[];
    // BULK: the ring comes first (16-byte aligned slots of one row each), then the slot barriers
    const uint32_t rowBytes = static_cast<uint32_t>(win) * sizeof(T);
    const int32_t ringSlots = BULK ? ringGroups * PF : 0;
    unsigned char* ring = reinterpret_cast<unsigned char*>(smemAll);
    uint64_t* bars = reinterpret_cast<uint64_t*>(ring + static_cast<size_t>(ringSlots) * rowBytes);
    float* smemF = reinterpret_cast<float*>(bars + ((ringSlots + 1) & ~1));
    const int32_t winPad = ParkedRowFloats(win);
    float* rowbufs = smemF;                                           // [kFlushBatch][winPad]
    float4* msm = reinterpret_cast<float4*>(smemF + kFlushBatch * winPad); // [metaRows][2]
    float* wsm = reinterpret_cast<float*>(msm + 2 * metaRows);        // [wTaps][wout]
    const int64_t p = blockIdx.x;
    const int32_t i0 = blockIdx.y * bandRows, i1 = min(hout, i0 + bandRows);
    const int32_t rlo = __ldg(th.xmin + i0);
    const int32_t rhi = min(__ldg(th.xmin + i1 - 1) + __ldg(th.xsize + i1 - 1), rlo + metaRows);
    // Column ownership: 16-byte load l of a thread covers columns l * (blockDim.x * LV) + threadIdx.x * LV ..,
    // so every load instruction of a warp reads one contiguous 512-byte run.
    const int32_t groupSpan = blockDim.x * LV;
    const int32_t c = threadIdx.x * LV;
    T* yp = y + p * hout * static_cast<int64_t>(wout);

    for (int32_t e = threadIdx.x; e < 2 * (rhi - rlo); e += blockDim.x) {
        msm[e] = __ldg(reinterpret_cast<const float4*>(wrow) + static_cast<int64_t>(rlo) * 2 + e);
    }
    for (int32_t j = threadIdx.x; j < wout && wTaps > 0; j += blockDim.x) {
        const int32_t n = min(__ldg(tw.xsize + j), wTaps);
        for (int32_t t = 0; t < n; ++t) {
            wsm[t * wout + j] = __ldg(tw.w + static_cast<int64_t>(j) * tw.taps + t);
        }
    }
    __syncthreads();

    float acc[kSlots][VC];
#pragma unroll
    for (int a = 0; a < kSlots; ++a) {
#pragma unroll
        for (int k = 0; k < VC; ++k) {
            acc[a][k] = 0.0f;
        }
    }
    // Completed output rows (vertical results, taken from the oldest accumulator slot) are parked in shared memory,
    // kFlushBatch rows at a time, and the horizontal filter then runs over the whole batch: a thread takes one
    // output column of all the batch's rows, so every weight is loaded once per batch and the rows give
    // independent accumulation chains. Output rows complete in increasing order, so a batch is rows
    // batchRow0 .. batchRow0 + pending - 1.
    int32_t pending = 0, batchRow0 = 0;
    auto runBatch = [&]() {
        __syncthreads(); // the batch's rows are written
        for (int32_t j = threadIdx.x; j < wout; j += blockDim.x) {
            const int32_t m = __ldg(tw.xmin + j), n = __ldg(tw.xsize + j);
            const float* wj = tw.w + static_cast<int64_t>(j) * tw.taps;
            float v[kFlushBatch];
#pragma unroll
            for (int bb = 0; bb < kFlushBatch; ++bb) {
                v[bb] = 0.0f;
            }
            // rows past `pending` hold stale values; their sums are not stored
            if (wTaps > 0) {
                const float* wp = wsm + j;
#pragma unroll 4
                for (int32_t t = 0; t < n; ++t) {
                    const float w = wp[t * wout];
                    const float* xr = rowbufs + Skew(m + t);
#pragma unroll
                    for (int bb = 0; bb < kFlushBatch; ++bb) {
                        v[bb] = fmaf(w, xr[bb * winPad], v[bb]);
                    }
                }
            } else {
                for (int32_t t = 0; t < n; ++t) {
                    const float w = __ldg(wj + t);
                    const float* xr = rowbufs + Skew(m + t);
#pragma unroll
                    for (int bb = 0; bb < kFlushBatch; ++bb) {
                        v[bb] = fmaf(w, xr[bb * winPad], v[bb]);
                    }
                }
            }
#pragma unroll
            for (int bb = 0; bb < kFlushBatch; ++bb) {
                if (bb < pending) {
                    yp[static_cast<int64_t>(batchRow0 + bb) * wout + j] = DType<T>::FromF(v[bb]);
                }
            }
        }
        __syncthreads(); // the rows have been read: the buffer can take the next batch
        pending = 0;
    };
    auto flush = [&](int32_t i) {
        if (pending == 0) {
            batchRow0 = i;
        }
        float* rowbuf = rowbufs + pending * winPad;
#pragma unroll
        for (int k = 0; k < VC; k += 4) {
            const int32_t col = (k / LV) * groupSpan + c + k % LV;
            if (col < win) { // four scalar stores: under the skew they are conflict-free across the warp
                const int32_t sc = Skew(col); // col is a multiple of 4: its four columns share one skew
                rowbuf[sc] = acc[0][k];
                rowbuf[sc + 1] = acc[0][k + 1];
                rowbuf[sc + 2] = acc[0][k + 2];
                rowbuf[sc + 3] = acc[0][k + 3];
            }
        }
        if (++pending == kFlushBatch) {
            runBatch();
        }
    };
    auto shift = [&]() {
#pragma unroll
        for (int a = 0; a + 1 < kSlots; ++a) {
#pragma unroll
            for (int k = 0; k < VC; ++k) {
                acc[a][k] = acc[a + 1][k];
            }
        }
#pragma unroll
        for (int k = 0; k < VC; ++k) {
            acc[kSlots - 1][k] = 0.0f;
        }
    };
    // Input rows are fetched PF rows ahead into fixed registers (the row loop is unrolled by PF; rotating a queue
    // through moves would make every iteration wait for the newest load), or ringGroups groups ahead into the ring.
    using Vec = Pack<T, LV>;
    Vec q[PF][NL];
    const T* xrows = x + (p * hin + rlo) * static_cast<int64_t>(win); // row rlo of this plane
    const T* xnext = xrows + c;                                       // next row to fetch (register path)
    int32_t rnext = rlo;
    auto fetch = [&](Vec (&dst)[NL]) {
        if (rnext < rhi) {
#pragma unroll
            for (int l = 0; l < NL; ++l) {
                if (l * groupSpan + c < win) {
                    dst[l] = *reinterpret_cast<const Vec*>(xnext + l * groupSpan);
                }
            }
        }
        xnext += win;
        ++rnext;
    };
    // BULK: thread 0 starts the copies of group `grp` (rows rlo + grp * PF ..) into the group's slots
    auto issueGroup = [&](int32_t grp) {
        const int32_t slot0 = (grp % ringGroups) * PF;
#pragma unroll
        for (int f = 0; f < PF; ++f) {
            const int32_t rr = grp * PF + f; // row index relative to rlo
            if (rlo + rr < rhi) {
                BulkLoadRow(ring + static_cast<size_t>(slot0 + f) * rowBytes, xrows + static_cast<int64_t>(rr) * win,
                            rowBytes, bars + slot0 + f);
            }
        }
    };
    if (BULK) {
        if (threadIdx.x == 0) {
            for (int32_t sl = 0; sl < ringSlots; ++sl) {
                BarrierInit(bars + sl, 1);
            }
            BarrierInitFence();
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int32_t grp = 0; grp < ringGroups; ++grp) {
                issueGroup(grp);
            }
        }
    } else {
#pragma unroll
        for (int f = 0; f < PF; ++f) {
            fetch(q[f]);
        }
    }
    int32_t curStart = __float_as_int(msm[1].z);
    for (int32_t r0 = rlo; r0 < rhi; r0 += PF) {
        const int32_t grp = (r0 - rlo) / PF;
        const int32_t slot0 = BULK ? (grp % ringGroups) * PF : 0;
        if (BULK) {
            // wait for the rows of this group; the outcome is made uniform so that the block leaves together
            const uint32_t parity = static_cast<uint32_t>(grp / ringGroups) & 1u;
            bool ok = true;
#pragma unroll
            for (int f = 0; f < PF; ++f) {
                if (r0 + f < rhi) {
                    ok = BarrierWait(bars + slot0 + f, parity, kWaitLimit) && ok;
                }
            }
            if (__syncthreads_or(!ok)) {
                if (threadIdx.x == 0) {
                    atomicAdd(&g_asyncCopyTimeouts, 1u);
                    // copies still in flight target this block's shared memory: give them a bounded chance to land
                    for (int32_t g2 = grp; g2 < grp + ringGroups; ++g2) {
                        for (int f = 0; f < PF; ++f) {
                            if (rlo + g2 * PF + f < rhi) {
                                BarrierWait(bars + (g2 % ringGroups) * PF + f,
                                            static_cast<uint32_t>(g2 / ringGroups) & 1u, 1u << 16);
                            }
                        }
                    }
                }
                return;
            }
        }
#pragma unroll
        for (int f = 0; f < PF; ++f) {
            const int32_t r = r0 + f;
            if (r < rhi) {
                const float4 m0 = msm[2 * (r - rlo)], m1 = msm[2 * (r - rlo) + 1];
                const int32_t s = __float_as_int(m1.z), cnt = __float_as_int(m1.w);
                while (curStart < s) { // outputs before start(r) no longer receive rows: complete
                    if (curStart >= i0 && curStart < i1) {
                        flush(curStart);
                    }
                    shift();
                    ++curStart;
                }
                const float w[kSlots] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y};
                float xv[VC];
                if (BULK) {
                    const T* srow = reinterpret_cast<const T*>(ring + static_cast<size_t>(slot0 + f) * rowBytes);
#pragma unroll
                    for (int l = 0; l < NL; ++l) {
                        Vec v{};
                        if (l * groupSpan + c < win) {
                            v = *reinterpret_cast<const Vec*>(srow + l * groupSpan + c);
                        }
                        float part[LV];
                        UnpackToF<T, LV>(v, part);
#pragma unroll
                        for (int k = 0; k < LV; ++k) {
                            xv[l * LV + k] = part[k];
                        }
                    }
                } else {
#pragma unroll
                    for (int l = 0; l < NL; ++l) {
                        float part[LV];
                        UnpackToF<T, LV>(q[f][l], part);
#pragma unroll
                        for (int k = 0; k < LV; ++k) {
                            xv[l * LV + k] = part[k];
                        }
                    }
                }
#pragma unroll
                for (int a = 0; a < kSlots; ++a) {
                    if (a < cnt) { // slots past the run are not touched (an Inf / NaN input must not leak in)
#pragma unroll
                        for (int k = 0; k < VC; ++k) {
                            acc[a][k] = fmaf(w[a], xv[k], acc[a][k]);
                        }
                    }
                }
                if (!BULK) {
                    fetch(q[f]);
                }
            }
        }
        if (BULK) {
            __syncthreads(); // every thread has read the group's slots: they can be refilled
            if (threadIdx.x == 0 && rlo + (grp + ringGroups) * PF < rhi) {
                issueGroup(grp + ringGroups);
            }
        }
    }
    const int32_t lastEnd = __float_as_int(msm[2 * (rhi - 1 - rlo) + 1].z) + __float_as_int(msm[2 * (rhi - 1 - rlo) + 1].w);
    while (curStart < i1 && curStart < lastEnd) {
        if (curStart >= i0) {
            flush(curStart);
        }
        shift();
        ++curStart;
    }
    if (pending > 0) {
        runBatch();
    }
}

// ---- backward, gather (direct) --------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
    AABwdGatherKernel(const T* __restrict__ go, T* __restrict__ gi, int32_t hin, int32_t win, int32_t hout,
                      int32_t wout, AAAxis th, AAAxis tw, RangeAxis rh, RangeAxis rw, int64_t total)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t row = idx / win;
        const int32_t x = static_cast<int32_t>(idx - row * win);
        const int64_t p = row / hin;
        const int32_t y = static_cast<int32_t>(row - p * hin);
        const int32_t is = __ldg(rh.start + y), ie = __ldg(rh.end + y);
        const int32_t js = __ldg(rw.start + x), je = __ldg(rw.end + x);
        const T* gp = go + p * hout * static_cast<int64_t>(wout);
        float value = 0.0f;
        for (int32_t i = is; i < ie; ++i) {
            const int32_t ty = y - __ldg(th.xmin + i);
            if (ty < 0 || ty >= __ldg(th.xsize + i)) {
                continue;
            }
            const float weightH = __ldg(th.w + static_cast<int64_t>(i) * th.taps + ty);
            if (weightH == 0.0f) {
                continue;
            }
            const T* gr = gp + static_cast<int64_t>(i) * wout;
            for (int32_t j = js; j < je; ++j) {
                const int32_t tx = x - __ldg(tw.xmin + j);
                if (tx < 0 || tx >= __ldg(tw.xsize + j)) {
                    continue;
                }
                const float weightW = __ldg(tw.w + static_cast<int64_t>(j) * tw.taps + tx);
                if (weightW == 0.0f) {
                    continue;
                }
                value = Add(value, Mul(Mul(DType<T>::Load(gr + j), weightH), weightW));
            }
        }
        gi[idx] = DType<T>::FromF(value);
    }
}

// ---- backward, band-tiled (down-scaling forward) ----------------------------------------------------------------
// gi[y][x] = sum_i wH(i,y) * sum_j wW(j,x) * go[i][j]. For scale >= 1 only a few outputs cover any input row or
// column, so the sum is done separably per block: the grads rows feeding a band of grad_input rows are staged in
// shared memory (fp32); for kBwdRows grad_input rows at a time the block first reduces vertically
// (t[y][j] = sum_i wH * go[i][j], one thread per (row, grads column)), then every thread expands horizontally for
// its four grad_input columns with the column weights it keeps in registers, and stores 16 bytes per row.
// Vertical and horizontal weights come from the slot tables built by AARowWeightKernel for both axes.
constexpr int kBwdRows = 4;   // grad_input rows per synchronisation
constexpr int kBwdColSlots = 8; // grads columns covering four consecutive grad_input columns (<= kSlots + 2)

template <typename T>
__global__ void __launch_bounds__(1024)
    AABwdBandKernel(const T* __restrict__ go, T* __restrict__ gi, int32_t hin, int32_t win, int32_t hout,
                    int32_t wout, RangeAxis rh, RangeAxis rw, const float* __restrict__ wrowH,
                    const float* __restrict__ wrowW, int32_t bandRows, int32_t stageRows)
{
    extern __shared__ __align__(16) float smemF[];
    float4* msm = reinterpret_cast<float4*>(smemF);            // [bandRows][2] vertical slot records of the band's rows
    float* gos = smemF + static_cast<int64_t>(bandRows) * 8;   // [stageRows][wout] grads rows of the band
    float* tbuf = gos + static_cast<int64_t>(stageRows) * wout; // [kBwdRows][wout]
    const int64_t p = blockIdx.x;
    const int32_t y0 = blockIdx.y * bandRows, y1 = min(hin, y0 + bandRows);
    for (int32_t e = threadIdx.x; e < 2 * (y1 - y0); e += blockDim.x) {
        msm[e] = __ldg(reinterpret_cast<const float4*>(wrowH) + static_cast<int64_t>(y0) * 2 + e);
    }
    const int32_t i0 = __ldg(rh.start + y0);
    const int32_t i1 = min(max(i0, __ldg(rh.end + y1 - 1)), i0 + stageRows);
    const T* gp = go + (p * hout + i0) * static_cast<int64_t>(wout);
    // While staging, note whether the band's grads rows hold an Inf / NaN: then the horizontal step takes a path that
    // only touches the sources covering each column, so that a non-finite value reaches exactly the columns it
    // reaches in the reference (the fast path multiplies uncovered sources by 0).
    bool sawNonFinite = false;
    for (int32_t e = threadIdx.x; e < (i1 - i0) * wout; e += blockDim.x) {
        const float v = DType<T>::Load(gp + e);
        gos[e] = v;
        sawNonFinite |= !(fabsf(v) <= 3.402823466e38f);
    }
    // horizontal weights of my four columns: slot u <-> grads column j0 + u
    const int32_t x = threadIdx.x * 4;
    const bool hasCols = x < win;
    int32_t j0 = 0;
    float wreg[4][kBwdColSlots];
    if (hasCols) {
        j0 = __ldg(rw.start + x);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int32_t sk = __ldg(rw.start + x + k), ek = __ldg(rw.end + x + k);
#pragma unroll
            for (int u = 0; u < kBwdColSlots; ++u) {
                const int32_t a = j0 + u - sk; // slot of grads column j0 + u in column x + k's own table
                wreg[k][u] = (a >= 0 && a < kSlots && j0 + u < ek)
                                 ? __ldg(wrowW + static_cast<int64_t>(x + k) * kSlotStride + a)
                                 : 0.0f;
            }
        }
    }
    const int32_t jcnt = hasCols ? min(kBwdColSlots, __ldg(rw.end + x + 3) - j0) : 0;
    const bool masked = __syncthreads_or(sawNonFinite) != 0; // also: the staged rows and records are visible
    T* op = gi + p * hin * static_cast<int64_t>(win);
    for (int32_t yb = y0; yb < y1; yb += kBwdRows) {
        // vertical: a thread takes one grads column for the kBwdRows rows of the step; the rows' slot records
        // (weights, first grads row, count) are block-uniform shared-memory reads
        for (int32_t j = threadIdx.x; j < wout; j += blockDim.x) {
#pragma unroll
            for (int ry = 0; ry < kBwdRows; ++ry) {
                const int32_t y = yb + ry;
                float v = 0.0f;
                if (y < y1) {
                    const float4 m0 = msm[2 * (y - y0)], m1 = msm[2 * (y - y0) + 1];
                    const int32_t s = __float_as_int(m1.z), cnt = __float_as_int(m1.w);
                    const float w[kSlots] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y};
                    const float* gcol = gos + (s - i0) * wout + j;
                    const int32_t run = min(cnt, i1 - s); // slots past the run (or past the staged rows) are not read
#pragma unroll
                    for (int a = 0; a < kSlots; ++a) {
                        if (a >= run) { // the same for every thread of the block
                            break;
                        }
                        v = fmaf(w[a], gcol[a * wout], v);
                    }
                }
                tbuf[ry * wout + j] = v;
            }
        }
        __syncthreads();
        if (hasCols) {
            T* dst = op + static_cast<int64_t>(yb) * win + x;
            const float* tr = tbuf + j0;
#pragma unroll
            for (int ry = 0; ry < kBwdRows; ++ry) {
                if (yb + ry < y1) {
                    float out[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    if (!masked) {
#pragma unroll
                        for (int u = 0; u < kBwdColSlots; ++u) {
                            if (u < jcnt) { // slots past the run are not read
                                const float t = tr[u];
#pragma unroll
                                for (int k = 0; k < 4; ++k) {
                                    out[k] = fmaf(wreg[k][u], t, out[k]);
                                }
                            }
                        }
                    } else { // same sums, but a source is only multiplied into the columns it covers
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int32_t sk = __ldg(rw.start + x + k), ek = __ldg(rw.end + x + k);
#pragma unroll
                            for (int u = 0; u < kBwdColSlots; ++u) {
                                if (u < jcnt && j0 + u >= sk && j0 + u < ek) {
                                    out[k] = fmaf(wreg[k][u], tr[u], out[k]);
                                }
                            }
                        }
                    }
                    StorePack<T, 4>(dst, out);
                }
                dst += win;
                tr += wout;
            }
        }
        __syncthreads();
    }
}

// ---- backward, atomic -------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
    AABwdAtomicKernel(const T* __restrict__ go, float* __restrict__ acc, int32_t hin, int32_t win, int32_t hout,
                      int32_t wout, AAAxis th, AAAxis tw, int64_t total)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t row = idx / wout;
        const int32_t w = static_cast<int32_t>(idx - row * wout);
        const int64_t p = row / hout;
        const int32_t h = static_cast<int32_t>(row - p * hout);
        const int32_t hmin = __ldg(th.xmin + h), hsz = __ldg(th.xsize + h);
        const int32_t wmin = __ldg(tw.xmin + w), wsz = __ldg(tw.xsize + w);
        const float* wh = th.w + static_cast<int64_t>(h) * th.taps;
        const float* ww = tw.w + static_cast<int64_t>(w) * tw.taps;
        const float v = DType<T>::Load(go + idx);
        float* ap = acc + p * hin * static_cast<int64_t>(win);
        for (int32_t m = 0; m < hsz; ++m) {
            const float weightH = __ldg(wh + m);
            if (weightH == 0.0f) {
                continue;
            }
            float* ar = ap + static_cast<int64_t>(hmin + m) * win + wmin;
            for (int32_t n = 0; n < wsz; ++n) {
                const float weightW = __ldg(ww + n);
                if (weightW == 0.0f) {
                    continue;
                }
                atomicAdd(ar + n, Mul(Mul(v, weightH), weightW));
            }
        }
    }
}

} // namespace

AAFwdPlan MakeAAFwdPlan(Dt dt, Shape4 sh, float scaleH, int32_t tapsW)
{
    AAFwdPlan plan{};
    // Streaming needs: every input row covered by at most kSlots outputs (true for scale >= 1), rows that one
    // block can own (8 columns per thread) and 16-byte aligned rows.
    const int es = DtSize(dt);
    plan.stream = scaleH >= 1.0f && sh.win % 8 == 0 && sh.win <= 8 * kStreamMaxThreads && (sh.win * es) % 16 == 0;
    if (!plan.stream) {
        return plan;
    }
    // fp32 rows of up to 1024 columns: four columns per thread (twice the warps of the 8-column variant at the same
    // number of resident blocks measured ~8 % faster); 16-bit rows and longer rows: eight columns (one or two
    // 16-byte loads per thread and row).
    plan.cols = (es == 4 && sh.win <= 4 * kStreamMaxThreads) ? 4 : 8;
    const int32_t threads = std::max(64, static_cast<int32_t>((CeilDiv(sh.win, plan.cols) + 31) & ~31));
    plan.threads = std::min(kStreamMaxThreads, threads);
    // Bands: pick the number of bands per plane whose block count fills whole waves of resident blocks best
    // (every band re-reads the input rows of its first window, so no more than 8, and at least 16 rows each).
    const int64_t planes = std::max<int64_t>(sh.n * sh.c, 1);
    const int64_t resident = static_cast<int64_t>(NumSMs()) * (plan.cols == 4 ? 4 : std::max(1, 512 / plan.threads));
    int64_t bestBands = 1;
    double bestEff = 0.0;
    for (int64_t b = 1; b <= 8 && sh.hout / b >= 16; ++b) {
        const int64_t blocks = planes * b;
        const double eff = static_cast<double>(blocks) / (static_cast<double>(CeilDiv(blocks, resident)) * resident);
        if (eff > bestEff + 0.02) {
            bestEff = eff;
            bestBands = b;
        }
    }
    plan.bandRows = static_cast<int32_t>(CeilDiv(sh.hout, bestBands));
    // input rows of a band: its windows span bandRows * scale + 2 * support (+ rounding) rows
    plan.metaRows = static_cast<int32_t>(
        std::min<double>(sh.hin, std::ceil(static_cast<double>(plan.bandRows) * scaleH + 4.0 * scaleH + 4.0)));
    // horizontal weights in shared memory if they fit beside the row buffer and the slot records
    const size_t wBytes = static_cast<size_t>(tapsW) * sh.wout * sizeof(float);
    const size_t rest = (kFlushBatch * static_cast<size_t>(ParkedRowFloats(sh.win)) + static_cast<size_t>(plan.metaRows) * 8 + 8) * sizeof(float);
    plan.regWeights = wBytes + rest <= 96 * 1024;
    if (rest > 96 * 1024) {
        plan.stream = false;
    }
    plan.wrowBytes = static_cast<uint64_t>(sh.hin) * kSlotStride * sizeof(float);
    // The bulk-copy row ring is off by default: on B200 it measured 15-25 % slower than register prefetch for this
    // kernel (the limiter is the shared-memory data pipe of the horizontal pass, not load latency, and the ring adds
    // shared-memory traffic and two block barriers per four rows). OPSCV_AA_RING=<groups> (2..4) selects it.
    plan.ringGroups = 0;
    if (const char* o = getenv("OPSCV_AA_RING")) {
        const int groups = atoi(o);
        const size_t ring = static_cast<size_t>(groups) * 4 * sh.win * es + 64;
        const size_t used = rest + (plan.regWeights ? wBytes : 0);
        if (groups >= 2 && groups <= 4 && used + ring <= 200 * 1024) {
            plan.ringGroups = groups;
        }
    }
    return plan;
}

uint32_t AsyncCopyTimeouts()
{
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_asyncCopyTimeouts, sizeof(v)) != cudaSuccess) {
        return 0xffffffffu;
    }
    return v;
}

cudaError_t BicubicAAFwd(Dt dt, const void* x, void* y, Shape4 sh, AAAxis th, AAAxis tw, RangeAxis rh,
                         float* wrow, const AAFwdPlan& plan, cudaStream_t s)
{
    const int64_t planes = sh.n * sh.c;
    const bool stream = plan.stream && Aligned(x, 16) && planes < (1LL << 31) && CeilDiv(sh.hout, plan.bandRows) <= 65535;
    if (stream) {
        AARowWeightKernel<<<static_cast<unsigned>(CeilDiv(sh.hin, 128)), 128, 0, s>>>(th, rh, sh.hin, wrow);
        const dim3 grid(static_cast<unsigned>(planes), static_cast<unsigned>(CeilDiv(sh.hout, plan.bandRows)));
        const int32_t wTaps = plan.regWeights ? tw.taps : 0;
        const size_t base = (kFlushBatch * static_cast<size_t>(ParkedRowFloats(sh.win)) + static_cast<size_t>(plan.metaRows) * 8 +
                             static_cast<size_t>(wTaps) * sh.wout) * sizeof(float);
        cudaError_t e = cudaSuccess;
        OPSCV_DISPATCH_DT(dt, T, {
            const T* px = static_cast<const T*>(x);
            T* py = static_cast<T*>(y);
            const int32_t slots = plan.ringGroups * 4;
            const size_t smem = base + (plan.ringGroups > 0 ? static_cast<size_t>(slots) * sh.win * sizeof(T) +
                                                                  static_cast<size_t>((slots + 1) & ~1) * 8
                                                            : 0);
            auto launch = [&](auto kernel) {
                if (smem > 48 * 1024) {
                    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(smem));
                }
                if (e == cudaSuccess) {
                    kernel<<<grid, plan.threads, smem, s>>>(px, py, sh.hin, sh.win, sh.hout, sh.wout, th, tw, wrow,
                                                            plan.bandRows, plan.metaRows, wTaps, plan.ringGroups);
                }
            };
            if (plan.cols == 4) {
                if constexpr (sizeof(T) == 4) {
                    if (plan.ringGroups > 0) {
                        launch(AAFwdStreamKernel<T, 4, kStreamMaxThreads, true>);
                    } else {
                        launch(AAFwdStreamKernel<T, 4, kStreamMaxThreads, false>);
                    }
                }
            } else if (plan.ringGroups > 0) {
                launch(AAFwdStreamKernel<T, 8, kStreamMaxThreads, true>);
            } else {
                launch(AAFwdStreamKernel<T, 8, kStreamMaxThreads, false>);
            }
        });
        CountLaunch(2);
        return e != cudaSuccess ? e : cudaGetLastError();
    }
    const int64_t total = planes * sh.hout * static_cast<int64_t>(sh.wout);
    OPSCV_DISPATCH_DT(dt, T, {
        AAFwdDirectKernel<T><<<GridFor(total, kThreads), kThreads, 0, s>>>(
            static_cast<const T*>(x), static_cast<T*>(y), sh.hin, sh.win, sh.hout, sh.wout, th, tw, total);
    });
    CountLaunch();
    return cudaGetLastError();
}

// Shared memory of one block of the band kernel: slot records of the band's rows, staged grads rows, step buffer.
static size_t AABwdSmem(int32_t bandRows, int32_t stageRows, int32_t wout)
{
    return (static_cast<size_t>(bandRows) * 8 + (static_cast<size_t>(stageRows) + kBwdRows) * wout) * sizeof(float);
}

AABwdPlan MakeAABwdPlan(Dt dt, Shape4 sh, float scaleH, float scaleW)
{
    AABwdPlan plan{};
    const int es = DtSize(dt);
    // Same covering bound as the forward streaming kernel, on both axes; one block owns whole grad_input rows.
    plan.band = scaleH >= 1.0f && scaleW >= 1.0f && sh.win % 4 == 0 && sh.win <= 4096 && (sh.win * es) % 8 == 0;
    if (!plan.band) {
        return plan;
    }
    plan.threads = std::min(1024, std::max(128, static_cast<int32_t>((CeilDiv(sh.win, 4) + 31) & ~31)));
    // Bands per plane: the split whose blocks fill whole waves of resident blocks best (up to four 256-thread
    // blocks per SM, fewer if the staged grads rows need more shared memory). t grad_input rows are fed by at most
    // t / scale + kSlots + 2 grads rows.
    const int64_t planes = std::max<int64_t>(sh.n * sh.c, 1);
    double bestScore = 0.0;
    for (int32_t b = 1; b <= 64 && (b == 1 || sh.hin / b >= 4 * kBwdRows); ++b) {
        int32_t band = static_cast<int32_t>(CeilDiv(sh.hin, b));
        band = (band + kBwdRows - 1) / kBwdRows * kBwdRows;
        const int32_t stage = static_cast<int32_t>(
            std::min<int64_t>(static_cast<int64_t>(band / static_cast<double>(scaleH)) + kSlots + 2, sh.hout));
        const size_t smem = AABwdSmem(band, stage, sh.wout);
        if (smem > 200 * 1024) {
            continue;
        }
        const int64_t perSm = std::min<int64_t>({4, 2048 / plan.threads, static_cast<int64_t>((225 * 1024) / (smem + 1024))});
        const int64_t slots = static_cast<int64_t>(NumSMs()) * std::max<int64_t>(perSm, 1);
        const int64_t blocks = planes * CeilDiv(sh.hin, band);
        // waves filled, times the residency reached, with a slight preference for fewer (taller) bands
        const double score = static_cast<double>(blocks) / (static_cast<double>(CeilDiv(blocks, slots)) * slots) *
                             (0.5 + 0.125 * static_cast<double>(perSm)) - 0.001 * b;
        if (score > bestScore) {
            bestScore = score;
            plan.bandRows = band;
            plan.stageRows = stage;
        }
    }
    if (bestScore <= 0.0) {
        plan.band = false;
        return plan;
    }
    plan.wrowBytesH = static_cast<uint64_t>(sh.hin) * kSlotStride * sizeof(float);
    plan.wrowBytesW = static_cast<uint64_t>(sh.win) * kSlotStride * sizeof(float);
    return plan;
}

cudaError_t BicubicAABwdGather(Dt dt, const void* go, void* gi, Shape4 sh, AAAxis th, AAAxis tw, RangeAxis rh,
                               RangeAxis rw, float* wrowH, float* wrowW, const AABwdPlan& plan, cudaStream_t s)
{
    const int64_t planes = sh.n * sh.c;
    const bool band = plan.band && Aligned(gi, 16) && planes < (1LL << 31) && CeilDiv(sh.hin, plan.bandRows) <= 65535;
    if (band) {
        AARowWeightKernel<<<static_cast<unsigned>(CeilDiv(sh.hin, 128)), 128, 0, s>>>(th, rh, sh.hin, wrowH);
        AARowWeightKernel<<<static_cast<unsigned>(CeilDiv(sh.win, 128)), 128, 0, s>>>(tw, rw, sh.win, wrowW);
        const dim3 grid(static_cast<unsigned>(planes), static_cast<unsigned>(CeilDiv(sh.hin, plan.bandRows)));
        const size_t smem = AABwdSmem(plan.bandRows, plan.stageRows, sh.wout);
        cudaError_t e = cudaSuccess;
        OPSCV_DISPATCH_DT(dt, T, {
            if (smem > 48 * 1024) {
                e = cudaFuncSetAttribute(AABwdBandKernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
            }
            if (e == cudaSuccess) {
                AABwdBandKernel<T><<<grid, plan.threads, smem, s>>>(static_cast<const T*>(go), static_cast<T*>(gi), sh.hin,
                                                                   sh.win, sh.hout, sh.wout, rh, rw, wrowH, wrowW,
                                                                   plan.bandRows, plan.stageRows);
            }
        });
        CountLaunch(3);
        return e != cudaSuccess ? e : cudaGetLastError();
    }
    const int64_t total = planes * sh.hin * static_cast<int64_t>(sh.win);
    OPSCV_DISPATCH_DT(dt, T, {
        AABwdGatherKernel<T><<<GridFor(total, kThreads), kThreads, 0, s>>>(
            static_cast<const T*>(go), static_cast<T*>(gi), sh.hin, sh.win, sh.hout, sh.wout, th, tw, rh, rw, total);
    });
    CountLaunch();
    return cudaGetLastError();
}

cudaError_t BicubicAABwdAtomic(Dt dt, const void* go, void* gi, float* acc, Shape4 sh, AAAxis th, AAAxis tw,
                               cudaStream_t s)
{
    const int64_t outElems = sh.n * sh.c * sh.hin * static_cast<int64_t>(sh.win);
    const int64_t total = sh.n * sh.c * sh.hout * static_cast<int64_t>(sh.wout);
    cudaError_t e = cudaMemsetAsync(acc, 0, static_cast<size_t>(outElems) * sizeof(float), s);
    if (e != cudaSuccess) {
        return e;
    }
    OPSCV_DISPATCH_DT(dt, T, {
        AABwdAtomicKernel<T><<<GridFor(total, kThreads), kThreads, 0, s>>>(static_cast<const T*>(go), acc, sh.hin,
                                                                           sh.win, sh.hout, sh.wout, th, tw, total);
    });
    CountLaunch(2);
    e = cudaGetLastError();
    if (e != cudaSuccess) {
        return e;
    }
    if (dt != Dt::F32 || static_cast<void*>(acc) != gi) {
        return CastFromF32(dt, gi, acc, outElems, s);
    }
    return cudaSuccess;
}

} // namespace opscv
