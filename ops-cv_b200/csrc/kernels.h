// Host-callable launchers of the CUDA kernels. Plain C++ (no CUDA types beyond cudaStream_t / cudaError_t) so
// that the aclnn host layer can be compiled as ordinary C++.
#pragma once

#include <cuda_runtime_api.h>
#include <stdint.h>

namespace opscv {

enum class Dt : int32_t { F32 = 0, F16 = 1, BF16 = 2 };
inline int DtSize(Dt d) { return d == Dt::F32 ? 4 : 2; }

enum Layout : int32_t { kNCHW = 0, kNHWC = 1 };

// Per-thread launch counter (incremented by every kernel launch made through these launchers).
void CountLaunch(int n = 1);
uint64_t LaunchCount();
void ResetLaunchCount();

// ---- per-axis tables (device memory, normally carved out of the caller's workspace) ---------------------------
struct NearestAxis { // one entry per OUTPUT index
    int32_t* src;
};
struct RangeAxis { // one entry per grad_input index: window [start, end) of grad_output indices
    int32_t* start;
    int32_t* end;
};
struct LerpAxis { // one entry per output (forward) / grad_output (backward) index
    int32_t* lo;
    int32_t* hi;
    float* delta;
};
struct AAAxis { // one entry per output index; w is [out][taps], zero padded, already normalised
    int32_t* xmin;
    int32_t* xsize;
    float* w;
    int32_t taps;
};

struct AxisGeom {
    int32_t in;  // extent on the forward-input side (grad_input side for backward ops)
    int32_t out; // extent on the forward-output side
    float scale; // forward source-coordinate scale as the reference's tiling computes it
    // Nearest tables only: 1 selects the UpsampleNearestExact2d index rules (forward: floor((d + 0.5) * scale);
    // backward: `scale` is then the grads-per-grad_input ratio and the window starts at ceil(y * scale - 0.5)).
    int32_t exact = 0;
};

// Table builders (tables.cu). Each fills the H and the W table in one launch.
cudaError_t BuildNearestFwdTables(AxisGeom h, AxisGeom w, NearestAxis th, NearestAxis tw, cudaStream_t s);
cudaError_t BuildNearestBwdTables(AxisGeom h, AxisGeom w, RangeAxis th, RangeAxis tw, cudaStream_t s);
// variant 0 = forward kernel's formula, 1 = backward (scatter-definition) formula.
cudaError_t BuildLerpTables(AxisGeom h, AxisGeom w, bool halfPixel, int variant, LerpAxis th, LerpAxis tw,
                            cudaStream_t s);
// For every grad_input index y: [first, first+count) = the grad_output indices i with lo[i] == y or hi[i] == y.
// Backward tables (variant 1) and their ranges in one launch.
cudaError_t BuildLerpBwdTablesAndRanges(AxisGeom h, AxisGeom w, bool halfPixel, LerpAxis th, LerpAxis tw, RangeAxis rh,
                                        RangeAxis rw, cudaStream_t s);
cudaError_t BuildLerpBwdRanges(AxisGeom h, AxisGeom w, LerpAxis th, LerpAxis tw, RangeAxis rh, RangeAxis rw,
                               cudaStream_t s);
// backward = true: centre rule of the reference's cubic backward kernel (0.5 when the scale is 0).
// filter: 0 Keys cubic (UpsampleBicubic2dAA), 1 triangle (UpsampleBilinear2dAA).
cudaError_t BuildAATables(AxisGeom h, AxisGeom w, float invH, float invW, float supH, float supW, AAAxis th,
                          AAAxis tw, bool backward, int filter, cudaStream_t s);
// For every forward-input index y: [start, end) = output indices whose window covers y.
cudaError_t BuildAABwdRanges(AxisGeom h, AxisGeom w, AAAxis th, AAAxis tw, RangeAxis rh, RangeAxis rw,
                             cudaStream_t s);

// ---- resampling kernels ----------------------------------------------------------------------------------
struct Shape4 {
    int64_t n, c;
    int32_t hin, win, hout, wout; // hin/win = forward input extent, hout/wout = forward output extent
};

// Launch plans are made in the first phase, on the host, from exact host copies of the index tables
// (host_tables.h), and frozen into the executor.
struct NearestPlan {
    enum Schedule : int32_t { kDirect = 0, kTiled = 1, kInteger = 2 };
    int32_t schedule;
    int32_t tileRows; // kTiled: output rows per block
    int32_t bandRows; // kTiled: most input rows any tile reads (sizes the shared-memory stage)
    int32_t rh, rw;   // kInteger: replication factors
};
NearestPlan MakeNearestFwdPlan(Dt dt, Layout lay, Shape4 sh, AxisGeom gh, AxisGeom gw);
NearestPlan MakeNearestBwdPlan(Dt dt, Layout lay, Shape4 sh, AxisGeom gh, AxisGeom gw);
bool NearestFwdUsesInteger(Dt dt, Layout lay, const void* x, const void* y, Shape4 sh, const NearestPlan& plan);
bool NearestBwdUsesInteger(Dt dt, Layout lay, const void* go, const void* gi, Shape4 sh, const NearestPlan& plan);
cudaError_t NearestFwd(Dt dt, Layout lay, const void* x, void* y, Shape4 sh, NearestAxis th, NearestAxis tw,
                       const NearestPlan& plan, cudaStream_t s);
cudaError_t NearestBwd(Dt dt, Layout lay, const void* go, void* gi, Shape4 sh, RangeAxis th, RangeAxis tw,
                       const NearestPlan& plan, cudaStream_t s);
// Element strides of an NCHW view (a dense tensor has the strides of its extents).
struct ViewStrides {
    int64_t n, c, h, w;
    int32_t chan; // C, to split a plane index into (n, c)
};
// Nearest forward for whole-number up-scales with a W factor of 2 on strided NCHW views with unit W strides
// (strided_forward.cu): rh = the H factor. Usable() checks the strides and alignments the kernel needs.
bool NearestFwdX2PitchUsable(Dt dt, const void* x, ViewStrides si, const void* y, ViewStrides so, Shape4 sh);
cudaError_t NearestFwdX2Pitch(Dt dt, const void* x, ViewStrides si, void* y, ViewStrides so, Shape4 sh, int32_t rh,
                              cudaStream_t s);
// The matching backward (rh x 2 window sums): `big` describes grad_output, `small_` grad_input.
bool NearestBwdX2PitchUsable(Dt dt, const void* go, ViewStrides big, const void* gi, ViewStrides small_, Shape4 sh);
cudaError_t NearestBwdX2Pitch(Dt dt, const void* go, ViewStrides big, void* gi, ViewStrides small_, Shape4 sh, int32_t rh,
                              cudaStream_t s);
struct BilinearPlan {
    enum Schedule : int32_t { kDirect = 0, kTiled = 1, kW2 = 2, kX2 = 3 }; // kX2: backward, 2x on both axes
    int32_t schedule;
    int32_t tileRows; // kTiled: output (forward) / grad_input (backward) rows per block
    int32_t bandRows; // kTiled: most rows of the other tensor any tile reads
    int32_t tapsW;    // kTiled backward: most grads columns feeding one grad_input column
    int32_t planesPerBlock; // kTiled: planes whose bands share one block's shared memory
    bool zeroTwins;         // backward: the tables hold clamped-border sources with a zero-weight twin tap
    // kW2 forward: the column weights repeat with period two from column 1 on (delta[w] == delta[w-2] for w >= 3),
    // so the kernel takes them as three scalars (column 0, even columns, odd columns) instead of table reads
    bool periodicW;
    float dxFirst, dxEven, dxOdd;
    // forward, 16-bit tensors: 24 minus the most significant bits any column weight or its complement has; a value
    // of T with at most this many significand bits times a weight is exact in fp32 (0: unknown, never assume it)
    int32_t weightSlack;
    // forward NHWC: the row table is the 2x pattern (row 0 from input row 0 alone, rows 2i + 1 and 2i + 2 from input rows
    // i and i + 1, the last row from the last input row alone), so the walk needs no row indices from the table
    bool rowsX2;
    // kX2 backward with periodicW: the four column weights shared by every grad_input column but the first and last
    float bw[4];
    int32_t rowStart1; // kX2 backward: first grads row feeding grad_input row 1 (0 or 1; every other row follows 2y-1)
    // what the tables are built from (filled by the plan makers): kernels that evaluate their own entries, and the
    // entry points that build the tables on demand, take it from here
    AxisGeom geomH, geomW;
    bool halfPixel;
};
BilinearPlan MakeBilinearFwdPlan(Dt dt, Layout lay, Shape4 sh, AxisGeom gh, AxisGeom gw, bool halfPixel);
BilinearPlan MakeBilinearBwdPlan(Dt dtIn, Layout lay, Shape4 sh, AxisGeom gh, AxisGeom gw, bool halfPixel);
// buildTables: th / tw are workspace that has not been filled; BilinearFwd fills it (plan.geomH / geomW, forward
// formula) unless the kernel it picks evaluates its own entries. false: the caller has built the tables.
// outPitch / inPitch (both or neither): output and input are NCHW views with these N, C and H pitches and unit W
// strides; only where BilinearFwdTakesPitch says the kernel the plan selects takes pitches (the 2x-width kernel does).
cudaError_t BilinearFwd(Dt dt, Layout lay, const void* x, void* y, Shape4 sh, LerpAxis th, LerpAxis tw,
                        const BilinearPlan& plan, cudaStream_t s, bool buildTables = false,
                        const ViewStrides* outPitch = nullptr, const ViewStrides* inPitch = nullptr);
bool BilinearFwdTakesPitch(Dt dt, Layout lay, const void* x, const void* y, Shape4 sh, const BilinearPlan& plan,
                           const ViewStrides& in, const ViewStrides& out);
// Gather backward: dtIn = grad_output dtype, dtOut = grad_input dtype.
// buildTables: as for BilinearFwd, with the backward formula and the ranges.
// gradsPitch: grad_output is an NCHW view with these N, C and H pitches and a unit W stride; only where
// BilinearBwdTakesPitch says the kernel the plan selects takes pitches (the 2x kernel does).
cudaError_t BilinearBwdGather(Dt dtIn, Dt dtOut, Layout lay, const void* go, void* gi, Shape4 sh, LerpAxis th,
                              LerpAxis tw, RangeAxis rh, RangeAxis rw, const BilinearPlan& plan, cudaStream_t s,
                              bool buildTables = false, const ViewStrides* gradsPitch = nullptr);
bool BilinearBwdTakesPitch(Dt dtIn, Dt dtOut, Layout lay, const void* go, const void* gi, Shape4 sh,
                           const BilinearPlan& plan, const ViewStrides& grads);
// Scatter backward with fp32 atomics into `acc` (fp32, N*C*hin*win, zeroed by this call). If dtOut is fp32 the
// caller passes acc == gi; otherwise a cast pass writes gi.
cudaError_t BilinearBwdAtomic(Dt dtIn, Dt dtOut, Layout lay, const void* go, void* gi, float* acc, Shape4 sh,
                              LerpAxis th, LerpAxis tw, cudaStream_t s);

struct AAFwdPlan {
    bool stream;        // streaming down-scale kernel (else one thread per output element)
    bool regWeights;    // horizontal weights of all output columns fit in shared memory
    int32_t metaRows;   // most input rows a band touches (sizes the shared slot-weight records)
    int32_t cols;       // input columns per thread of the streaming kernel (4 or 8)
    int32_t ringGroups; // > 0: rows arrive by bulk asynchronous copies into a shared ring of this many 4-row groups
    int32_t threads;    // block size of the streaming kernel
    int32_t bandRows;   // output rows per block
    uint64_t wrowBytes; // workspace for the per-input-row vertical weights
};
AAFwdPlan MakeAAFwdPlan(Dt dt, Shape4 sh, float scaleH, int32_t tapsW);
// rh (ranges of outputs covering each input row) and wrow are only used by the streaming kernel.
cudaError_t BicubicAAFwd(Dt dt, const void* x, void* y, Shape4 sh, AAAxis th, AAAxis tw, RangeAxis rh, float* wrow,
                         const AAFwdPlan& plan, cudaStream_t s);
// Bounded waits on asynchronous copies that ran out since the library was loaded (0 in a healthy run).
uint32_t AsyncCopyTimeouts();

struct AABwdPlan {
    bool band;         // band-tiled separable kernel (else one thread per grad_input element)
    int32_t threads;   // block size
    int32_t bandRows;  // grad_input rows per block
    int32_t stageRows; // grads rows staged in shared memory per block
    uint64_t wrowBytesH, wrowBytesW; // workspace for the per-row / per-column slot weights
};
AABwdPlan MakeAABwdPlan(Dt dt, Shape4 sh, float scaleH, float scaleW);
cudaError_t BicubicAABwdGather(Dt dt, const void* go, void* gi, Shape4 sh, AAAxis th, AAAxis tw, RangeAxis rh,
                               RangeAxis rw, float* wrowH, float* wrowW, const AABwdPlan& plan, cudaStream_t s);
cudaError_t BicubicAABwdAtomic(Dt dt, const void* go, void* gi, float* acc, Shape4 sh, AAAxis th, AAAxis tw,
                               cudaStream_t s);

// UpsampleBicubic2d without antialiasing. schedule: 0 general, 2 / 3 one input / one output pixel, 4 integer
// source positions (equal extents are a copy made by the host layer). The backward is a gather in a fixed order.
cudaError_t Bicubic2dFwd(Dt dt, Layout lay, const void* x, void* y, Shape4 sh, float scaleH, float scaleW,
                         bool halfPixel, int32_t schedule, cudaStream_t s);
cudaError_t Bicubic2dBwd(Dt dt, Layout lay, const void* go, void* gi, Shape4 sh, float scaleH, float scaleW,
                         float invH, float invW, bool align, cudaStream_t s);

// UpsampleNearest3d / UpsampleNearestExact3d. rows: forward planes * dout * ho, backward planes * di * hi, with
// planes = N * C for NCDHW (chan = 1) and N for NDHWC (chan = C). Forward scales are source-coordinate scales; the
// backward's are the window scales (grads extent per grad_input extent).
struct Nearest3dGeom {
    int64_t rows;
    int32_t di, hi, wi, dout, ho, wo, chan;
    float sd, sh, sw;
    int32_t exact;
    // whole-number up-scale factors per axis when the host has checked that every index (forward) or window
    // (backward) of the axis follows them, else 0; rw == 2 with rd, rh >= 1 selects the replicate / pool kernels
    int32_t rd = 0, rh = 0, rw = 0;
};
cudaError_t Nearest3dFwd(Dt dt, const void* x, void* y, Nearest3dGeom g, cudaStream_t s);
cudaError_t Nearest3dBwd(Dt dt, const void* go, void* gi, Nearest3dGeom g, cudaStream_t s);

// UpsampleTrilinear3d / UpsampleTrilinear3dBackward. rows and chan as for Nearest3dGeom; sd / sh / sw are the
// source-coordinate scales of the reference's tiling. loop (forward only): 0 full, 1 / 2 / 3 only D / H / W is
// resampled, 4 copy.
struct Trilinear3dGeom {
    int64_t rows;
    int32_t di, hi, wi, dout, ho, wo, chan;
    float sd, sh, sw;
    int32_t align;
    int32_t loop;
};
// Backward weight lists, one per grad_input index of each axis (0 D, 1 H, 2 W): the grad_output indices
// [start, start + count) feed it with weights w[index * taps + k]; taps is the longest list of the axis.
struct TrilinearBwdTables {
    int32_t* start[3];
    int32_t* count[3];
    float* w[3];
    int32_t taps[3];
};
// stage: fp32 scratch of Trilinear3dFwdWorkspace / Trilinear3dBwdWorkspace bytes (planes = N * C for NCDHW, N for
// NDHWC); the forward needs none for the one-axis loops and the copy.
uint64_t Trilinear3dFwdWorkspace(const Trilinear3dGeom& g, int64_t planes);
uint64_t Trilinear3dBwdWorkspace(const Trilinear3dGeom& g, int64_t planes);
cudaError_t Trilinear3dFwd(Dt dt, const void* x, void* y, float* stage, Trilinear3dGeom g, cudaStream_t s);
cudaError_t BuildTrilinearBwdTables(TrilinearBwdTables t, Trilinear3dGeom g, cudaStream_t s);
cudaError_t Trilinear3dBwd(Dt dt, const void* go, void* gi, float* stage, Trilinear3dGeom g, TrilinearBwdTables t,
                           cudaStream_t s);

struct GridShape {
    int64_t n, c;
    int32_t hin, win, hout, wout;
    int32_t interp, pad, align;
};
// Forward plan: windowed != 0 selects the tile-major kernel that stages, per output tile, the window of the input
// planes the tile's taps fall into. vectors > 0 selects the shared-memory staged kernel with that many 16-byte channel vectors per
// pixel; it needs recBytes of workspace for the per-sample source coordinates.
struct GridFwdPlan {
    int32_t vectors;
    uint64_t recBytes;
    int32_t windowed; // 1: the per-tile windowed kernel (fp32 planes too large for the staged kernel)
};
GridFwdPlan PlanGridSampler2DFwd(Dt dt, GridShape g);
cudaError_t GridSampler2DFwd(Dt dt, const void* x, const void* grid, void* y, GridShape g, const GridFwdPlan& plan,
                             void* workspace, cudaStream_t s);

// Workspace needs of the grid-sampler backward (bytes, 256-byte aligned pieces); see grid_sampler_grad.cu.
struct GridGradPlan {
    bool deterministic;
    bool wantInput, wantGrid;
    int32_t stagedGroup; // > 0: shared-memory staged kernel with this many channels per block
    int32_t detGridGroup;  // deterministic grad_grid from the staged kernel with per-group partials (0: per-sample kernel)
    uint64_t gridAccBytes; // staged kernel: fp32 (gix, giy) sums per sample (per group and sample with partials)
    uint64_t recBytes;   // staged kernels: per-sample source coordinates (last piece of the workspace)
    uint64_t accBytes;   // fp32 grad_input accumulator (16-bit dtypes, atomic mode)
    int32_t detChunks, detChunkSamples; // deterministic: chunks of the sample sequence filled in parallel
    bool detCursorSmem;   // deterministic fill: append positions fit shared memory
    int32_t detGatherGroup; // deterministic gather: channels per block with grad_output staged (0: global gather)
    uint64_t countBytes; // deterministic: append positions per chunk and segment starts
    uint64_t entryBytes; // deterministic: sorted (sample, weight) entries
    uint64_t total;
};
GridGradPlan PlanGridSampler2DBwd(Dt dt, GridShape g, bool deterministic, bool wantInput, bool wantGrid);
cudaError_t GridSampler2DBwd(Dt dt, const void* go, const void* x, const void* grid, void* gi, void* ggrid,
                             GridShape g, const GridGradPlan& plan, void* workspace, cudaStream_t s);

// ---- strided views -----------------------------------------------------------------------------------------
// GridSampler3D on NCDHW tensors; interp 0 bilinear, 1 nearest; pad 0 zeros, 1 border, 2 reflection.
struct Grid3dShape {
    int64_t n, c;
    int32_t di, hi, wi, dout, ho, wo;
    int32_t interp, pad, align;
    int32_t cl = 0; // 1: input, output and gradients are channels-last (NDHWC), contiguous
};
cudaError_t GridSampler3dFwd(Dt dt, const void* x, const void* grid, void* y, Grid3dShape g, cudaStream_t s);
cudaError_t GridSampler3dBwd(Dt dt, const void* go, const void* x, const void* grid, void* gi, void* ggrid, float* acc,
                             Grid3dShape g, bool wantInput, bool wantGrid, cudaStream_t s);

// out[b][c][r] = in[b][r][c] (elements of 2 or 4 bytes): the NCDHW <-> NDHWC change of the 3-D grid sampler.
cudaError_t TransposeBatched(int elemSize, const void* in, void* out, int64_t batch, int64_t rows, int64_t cols,
                             cudaStream_t s);

struct View4 {
    int64_t dim[4];
    int64_t stride[4]; // in elements
};
// dst (contiguous, dims = v.dim) <- src view, or the reverse when `toView` is true. elemSize 2 or 4.
cudaError_t StridedCopy(int elemSize, void* contiguous, void* viewBase, View4 v, bool toView, cudaStream_t s);
cudaError_t CopyBytes(void* dst, const void* src, uint64_t bytes, cudaStream_t s);
// dst[i] = (T)src[i] for fp32 src.
cudaError_t CastFromF32(Dt dt, void* dst, const float* src, int64_t n, cudaStream_t s);

} // namespace opscv
