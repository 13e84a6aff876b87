// Data-movement helpers: strided view <-> contiguous staging (what the reference does with its Contiguous and
// ViewCopy steps around every operator), device-to-device copies for the same-size shortcuts, and the final
// fp32 -> storage-dtype cast of the atomic backward paths.
#include <algorithm>

#include "launch_util.cuh"

namespace opscv {

namespace {

thread_local int g_numSMs = 0;
thread_local uint64_t g_launches = 0;

constexpr int kThreads = 256;

// One thread row of a block walks the rows (i0, i1, i2) of the view, whose offset is found once per row; a thread
// moves V adjacent elements of the row (V > 1 only for a unit innermost stride with aligned rows).
template <typename E, int V>
__global__ void __launch_bounds__(kThreads)
    StridedCopyKernel(E* __restrict__ contiguous, E* __restrict__ viewBase, View4 v, bool toView, int64_t rows)
{
    const int64_t t0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * V;
    if (t0 >= v.dim[3]) {
        return;
    }
    const bool small = rows <= 0x7fffffffLL;
    const int64_t rowStep = static_cast<int64_t>(gridDim.y) * blockDim.y;
    for (int64_t row = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y; row < rows; row += rowStep) {
        int64_t i0, i1, i2;
        if (small) { // 32-bit divisions (a row count below 2^31 bounds every extent)
            const uint32_t r = static_cast<uint32_t>(row), d2 = static_cast<uint32_t>(v.dim[2]),
                           d1 = static_cast<uint32_t>(v.dim[1]);
            const uint32_t q = r / d2, p = q / d1;
            i2 = r - q * d2;
            i1 = q - p * d1;
            i0 = p;
        } else {
            const int64_t q = row / v.dim[2];
            i2 = row - q * v.dim[2];
            i0 = q / v.dim[1];
            i1 = q - i0 * v.dim[1];
        }
        E* pv = viewBase + i0 * v.stride[0] + i1 * v.stride[1] + i2 * v.stride[2] + t0 * v.stride[3];
        E* pc = contiguous + row * v.dim[3] + t0;
        if (toView) {
            *reinterpret_cast<Pack<E, V>*>(pv) = *reinterpret_cast<const Pack<E, V>*>(pc);
        } else {
            *reinterpret_cast<Pack<E, V>*>(pc) = *reinterpret_cast<const Pack<E, V>*>(pv);
        }
    }
}

template <typename E>
void LaunchStridedCopy(E* contiguous, E* viewBase, const View4& v, bool toView, cudaStream_t s)
{
    const int64_t rows = v.dim[0] * v.dim[1] * v.dim[2];
    int vec = 1;
    if (v.stride[3] == 1) {
        for (int w = 16 / static_cast<int>(sizeof(E)); w > 1; w >>= 1) {
            if (v.dim[3] % w == 0 && v.stride[0] % w == 0 && v.stride[1] % w == 0 && v.stride[2] % w == 0 &&
                Aligned(contiguous, w * sizeof(E)) && Aligned(viewBase, w * sizeof(E))) {
                vec = w;
                break;
            }
        }
    }
    const RowLaunch rl = RowTiling(rows, CeilDiv(v.dim[3], static_cast<int64_t>(vec)), kThreads);
    OPSCV_DISPATCH_VEC(vec, V, {
        if constexpr (V * sizeof(E) <= 16) {
            StridedCopyKernel<E, V><<<rl.grid, rl.block, 0, s>>>(contiguous, viewBase, v, toView, rows);
        }
    });
}

// out[b][c][r] = in[b][r][c]: 32 x 32 tiles through shared memory (one padding column: no bank conflicts), so that
// both the reads and the writes of a warp are contiguous. block = (32, 8).
template <typename E>
__global__ void __launch_bounds__(256)
    TransposeKernel(const E* __restrict__ in, E* __restrict__ out, int64_t rows, int64_t cols, int64_t tilesR,
                    int64_t tilesC, int64_t tiles)
{
    __shared__ E tile[32][33];
    for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int64_t b = t / (tilesR * tilesC);
        const int64_t rem = t - b * tilesR * tilesC;
        const int64_t tr = rem / tilesC, tc = rem - tr * tilesC;
        const E* pin = in + b * rows * cols;
        E* pout = out + b * rows * cols;
        __syncthreads(); // the previous tile has been written out
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            const int64_t r = tr * 32 + threadIdx.y + j, c = tc * 32 + threadIdx.x;
            if (r < rows && c < cols) {
                tile[threadIdx.y + j][threadIdx.x] = pin[r * cols + c];
            }
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            const int64_t c = tc * 32 + threadIdx.y + j, r = tr * 32 + threadIdx.x;
            if (r < rows && c < cols) {
                pout[c * rows + r] = tile[threadIdx.x][threadIdx.y + j];
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) CastKernel(T* __restrict__ dst, const float* __restrict__ src, int64_t n)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        dst[i] = DType<T>::FromF(src[i]);
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
    CastVec4Kernel(T* __restrict__ dst, const float* __restrict__ src, int64_t groups)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < groups; i += stride) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(src) + i);
        const float vals[4] = {v.x, v.y, v.z, v.w};
        StorePack<T, 4>(dst + i * 4, vals);
    }
}

} // namespace

int NumSMs()
{
    if (g_numSMs == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) {
            g_numSMs = n;
        } else {
            (void)cudaGetLastError();
            return kNumSMsFallback;
        }
    }
    return g_numSMs;
}

void CountLaunch(int n) { g_launches += static_cast<uint64_t>(n); }
uint64_t LaunchCount() { return g_launches; }
void ResetLaunchCount() { g_launches = 0; }

cudaError_t StridedCopy(int elemSize, void* contiguous, void* viewBase, View4 v, bool toView, cudaStream_t s)
{
    const int64_t total = v.dim[0] * v.dim[1] * v.dim[2] * v.dim[3];
    if (total == 0) {
        return cudaSuccess;
    }
    if (elemSize == 4) {
        LaunchStridedCopy<uint32_t>(static_cast<uint32_t*>(contiguous), static_cast<uint32_t*>(viewBase), v, toView, s);
    } else {
        LaunchStridedCopy<uint16_t>(static_cast<uint16_t*>(contiguous), static_cast<uint16_t*>(viewBase), v, toView, s);
    }
    CountLaunch();
    return cudaGetLastError();
}

cudaError_t TransposeBatched(int elemSize, const void* in, void* out, int64_t batch, int64_t rows, int64_t cols,
                             cudaStream_t s)
{
    if (batch * rows * cols == 0) {
        return cudaSuccess;
    }
    const int64_t tilesR = CeilDiv(rows, 32), tilesC = CeilDiv(cols, 32), tiles = batch * tilesR * tilesC;
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(tiles, static_cast<int64_t>(NumSMs()) * 32));
    const dim3 block(32, 8, 1);
    if (elemSize == 4) {
        TransposeKernel<uint32_t><<<grid, block, 0, s>>>(static_cast<const uint32_t*>(in), static_cast<uint32_t*>(out),
                                                         rows, cols, tilesR, tilesC, tiles);
    } else {
        TransposeKernel<uint16_t><<<grid, block, 0, s>>>(static_cast<const uint16_t*>(in), static_cast<uint16_t*>(out),
                                                         rows, cols, tilesR, tilesC, tiles);
    }
    CountLaunch();
    return cudaGetLastError();
}

cudaError_t CopyBytes(void* dst, const void* src, uint64_t bytes, cudaStream_t s)
{
    if (bytes == 0 || dst == src) {
        return cudaSuccess;
    }
    CountLaunch();
    return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, s);
}

cudaError_t CastFromF32(Dt dt, void* dst, const float* src, int64_t n, cudaStream_t s)
{
    if (n == 0) {
        return cudaSuccess;
    }
    if (dt == Dt::F32) {
        return CopyBytes(dst, src, static_cast<uint64_t>(n) * 4, s);
    }
    const bool vec = n % 4 == 0 && Aligned(dst, 8) && Aligned(src, 16);
    if (dt == Dt::F16) {
        if (vec) {
            CastVec4Kernel<__half><<<GridFor(n / 4, kThreads), kThreads, 0, s>>>(static_cast<__half*>(dst), src, n / 4);
        } else {
            CastKernel<__half><<<GridFor(n, kThreads), kThreads, 0, s>>>(static_cast<__half*>(dst), src, n);
        }
    } else {
        if (vec) {
            CastVec4Kernel<__nv_bfloat16><<<GridFor(n / 4, kThreads), kThreads, 0, s>>>(
                static_cast<__nv_bfloat16*>(dst), src, n / 4);
        } else {
            CastKernel<__nv_bfloat16><<<GridFor(n, kThreads), kThreads, 0, s>>>(static_cast<__nv_bfloat16*>(dst), src,
                                                                                n);
        }
    }
    CountLaunch();
    return cudaGetLastError();
}

} // namespace opscv
