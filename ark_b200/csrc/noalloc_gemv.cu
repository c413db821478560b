// arkb_matvec_splitk_static: a skinny split-K matmul that allocates nothing.
//
// Some hosts cannot call cudaMalloc where they need this product: code running
// inside a CUDA-graph capture or a stream-ordered section that must not
// synchronise the device, real-time loops that pre-allocate everything at
// start-up, and plug-ins living inside a process whose memory pool is owned by
// someone else. For them this entry point computes
//     y[M, N] = x[M, K] . W[N, K]^T        (fp16 or bf16, fp32 accumulation)
// like the split-K form of the engine's Matmul stage, but keeps the fp32
// partial sums in a fixed array that is part of the library image instead of
// in a scratch allocation. The caller supplies only x, W and y (device memory).
//
// The scratch is kStaticScratchBytes (4 MiB) of device memory per GPU that
// loads the library, held until the process exits. A call needs
// splits * M * N * 4 bytes of it and is rejected when that does not fit.
// Every call on a device uses the same array: nothing in it has to start at
// zero (each call overwrites the partials it later reads), but two calls that
// overlap on the GPU (different streams, no ordering) would race on it.
// The first call on each device looks up the array's device address
// (cudaGetSymbolAddress); make that first call outside any stream capture.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <string>

#include "ark_b200.h"

namespace arkb {
void set_last_error(const std::string &msg);  // capi.cpp: what arkb_last_error() returns on this thread
}

namespace {

constexpr size_t kStaticScratchBytes = 4u << 20;
constexpr int kMaxRows = 16;      // rows of x (M)
constexpr int kMaxDevices = 64;

// File-scope scratch. In host code this name is only a handle for the runtime's
// symbol look-up, never an address to hand to a kernel.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// per-device address of g_static_scratch and SM count, filled on first use (atomics: the first calls on a device
// may come from several host threads; they all store the same values)
std::atomic<float *> g_scratch_addr[kMaxDevices];
std::atomic<int> g_num_sm[kMaxDevices];

__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// One warp per (output column n, k-range s): lanes stride the range with 16-byte
// loads of W and x, fp32 accumulate, shuffle reduce; partial[s][m][n] is written
// unrounded.
template <typename T, int MAXM>
__global__ void __launch_bounds__(256) matvec_partials(const T *__restrict__ x, const T *__restrict__ w, float *partial, int M,
                                                        int N, int K, int splits, int kper) {
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long item = warp; item < (long long)N * splits; item += nwarps) {
        const int n = (int)(item / splits), s = (int)(item % splits);
        const int k0 = s * kper, k1 = min(K, k0 + kper);
        float acc[MAXM];
#pragma unroll
        for (int m = 0; m < MAXM; ++m) acc[m] = 0.0f;
        const T *wr = w + (long long)n * K;
        for (int k = k0 + lane * 8; k < k1; k += 32 * 8) {  // K and kper are multiples of 8
            const uint4 wv = *reinterpret_cast<const uint4 *>(wr + k);
            const T *we = reinterpret_cast<const T *>(&wv);
#pragma unroll
            for (int m = 0; m < MAXM; ++m) {
                if (m < M) {
                    const uint4 xv = *reinterpret_cast<const uint4 *>(x + (long long)m * K + k);
                    const T *xe = reinterpret_cast<const T *>(&xv);
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[m] += to_f(we[i]) * to_f(xe[i]);
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MAXM; ++m) {
            float v = acc[m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && m < M) partial[((long long)s * M + m) * N + n] = v;
        }
    }
}

// y[m][n] = sum over k-ranges, in range order, rounded once.
template <typename T>
__global__ void matvec_finish(const float *partial, T *y, int M, int N, int splits) {
    const long long total = (long long)M * N;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < splits; ++s) acc += partial[(long long)s * total + e];
        y[e] = from_f<T>(acc);
    }
}

}  // namespace

extern "C" arkb_status arkb_matvec_splitk_static(const void *x, const void *w, void *y, int m, int n, int k, int dtype,
                                                 void *stream) {
    auto fail = [](arkb_status st, const std::string &msg) {
        arkb::set_last_error(msg);
        return st;
    };
    if (!x || !w || !y) return fail(ARKB_INVALID_USAGE, "null operand");
    if (dtype != 1 && dtype != 2) return fail(ARKB_UNSUPPORTED, "dtype must be 1 (fp16) or 2 (bf16)");
    if (m < 1 || m > kMaxRows) return fail(ARKB_INVALID_USAGE, "m must be between 1 and " + std::to_string(kMaxRows));
    if (n < 1 || k < 8 || k % 8) return fail(ARKB_INVALID_USAGE, "n must be positive and k a positive multiple of 8");
    if (((uintptr_t)x | (uintptr_t)w) & 15) return fail(ARKB_INVALID_USAGE, "x and w must be 16-byte aligned");
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(ARKB_GPU_ERROR, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(ARKB_UNSUPPORTED, "device ordinal out of range");
    if (!g_scratch_addr[dev].load(std::memory_order_acquire)) {
        // once per device, with that device current: the device address of the static array
        float *p = nullptr;
        e = cudaGetSymbolAddress((void **)&p, g_static_scratch);
        if (e != cudaSuccess || !p) return fail(ARKB_GPU_ERROR, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess || sms < 1) return fail(ARKB_GPU_ERROR, std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e));
        g_num_sm[dev].store(sms, std::memory_order_relaxed);
        g_scratch_addr[dev].store(p, std::memory_order_release);
    }
    const int num_sm = g_num_sm[dev].load(std::memory_order_relaxed);
    // k-ranges: enough warps to fill the GPU, each range a multiple of 256 elements (one 16-byte load per lane)
    int splits = 1;
    const long long want_warps = (long long)num_sm * 32;
    while (splits < 64 && (long long)n * splits < want_warps && k / (splits * 2) >= 256) splits *= 2;
    int kper = ((k + splits - 1) / splits + 255) / 256 * 256;
    splits = (k + kper - 1) / kper;
    const size_t need = (size_t)splits * m * n * sizeof(float);
    if (need > kStaticScratchBytes)
        return fail(ARKB_INVALID_USAGE, "problem needs " + std::to_string(need) + " bytes of scratch, the static array holds " +
                                            std::to_string(kStaticScratchBytes) + " (splits * m * n * 4 must fit)");
    float *scratch = g_scratch_addr[dev].load(std::memory_order_relaxed);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const long long items = (long long)n * splits;
    const int blocks = (int)((items + 7) / 8 < num_sm * 8 ? (items + 7) / 8 : num_sm * 8);
    if (dtype == 1)
        matvec_partials<__half, kMaxRows><<<blocks, 256, 0, st>>>((const __half *)x, (const __half *)w, scratch, m, n, k, splits, kper);
    else
        matvec_partials<__nv_bfloat16, kMaxRows><<<blocks, 256, 0, st>>>((const __nv_bfloat16 *)x, (const __nv_bfloat16 *)w, scratch,
                                                                          m, n, k, splits, kper);
    const long long total = (long long)m * n;
    const int fb = (int)((total + 255) / 256 < num_sm * 4 ? (total + 255) / 256 : num_sm * 4);
    if (dtype == 1) matvec_finish<__half><<<fb, 256, 0, st>>>(scratch, (__half *)y, m, n, splits);
    else matvec_finish<__nv_bfloat16><<<fb, 256, 0, st>>>(scratch, (__nv_bfloat16 *)y, m, n, splits);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(ARKB_GPU_ERROR, std::string("kernel launch: ") + cudaGetErrorString(e));
    return ARKB_OK;
}
