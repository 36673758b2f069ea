// mk_linear_static: a split-k linear layer whose scratch memory is a fixed array inside
// the library instead of an allocation.
//
// Some hosts of this library cannot allocate device memory at the point where they need
// a linear layer: an inference server that handed the whole GPU to its own arena at start
// up, or a latency-critical loop that must not run into the device-wide synchronisation
// cudaMalloc and cudaFree imply.  For them this one entry point computes
//     out[t][n] = bf16( sum_k x[t][k] * w[n][k] (+ residual[t][n]) )
// with the same arithmetic as the "linear" / "linear_with_residual" tasks of the
// megakernel (fp32 accumulation, one rounding), and touches no allocator at all: the
// caller passes inputs and outputs, the partial sums of the k-splits and the arrival
// counters live in `g_scratch` below.  Every GPU that loads the library holds that array
// (about 4 MB) until the process exits.
//
// All calls share the array.  Two calls that overlap on the GPU (different streams, or
// different host threads) race on it; callers must serialise them.  The counters are
// cleared at the start of every call, the partial sums are fully overwritten before they
// are read, so nothing a previous call left behind is ever consumed.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/b200mk.h"

namespace {

constexpr int kMaxTokens = MK_STATIC_MAX_TOKENS;
constexpr int kMaxN = MK_STATIC_MAX_N;
constexpr int kMaxK = MK_STATIC_MAX_K;
constexpr int kMaxSplits = 8;
constexpr int kRowsPerBlock = 64;
constexpr int kCounters = kMaxN / kRowsPerBlock;
// [counters: kCounters u32, padded to 4 KB][partials: kMaxSplits x kMaxTokens x kMaxN floats]
constexpr size_t kCounterBytes = 4096;
constexpr size_t kScratchBytes = kCounterBytes + (size_t)kMaxSplits * kMaxTokens * kMaxN * sizeof(float);
static_assert(kCounters * sizeof(unsigned) <= kCounterBytes, "counter block too small");

// In host code this name is only a handle for cudaGetSymbolAddress; the device address
// it stands for is looked up once per device in scratch_for_current_device().
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
  f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
  f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
  f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}

// grid (row blocks of 64, k splits); 8 warps x 8 rows; a warp walks its k-slice in 16-byte steps
template <int T>
__global__ void __launch_bounds__(256) linear_static_kernel(const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ w,
                                                            const __nv_bfloat16* res, __nv_bfloat16* out, int n, int k,
                                                            int splits, unsigned char* scratch) {
  unsigned* counters = reinterpret_cast<unsigned*>(scratch);
  float* partial = reinterpret_cast<float*>(scratch + kCounterBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ks = blockIdx.y;
  const int kvec = k >> 3;
  const int per = (kvec + splits - 1) / splits;
  const int v0 = ks * per, v1 = min(kvec, v0 + per);
  for (int r = 0; r < 8; ++r) {
    const int row = blockIdx.x * kRowsPerBlock + warp * 8 + r;
    float acc[T];
#pragma unroll
    for (int t = 0; t < T; ++t) acc[t] = 0.f;
    if (row < n) {
      const uint4* wr = reinterpret_cast<const uint4*>(w + (size_t)row * k);
      for (int v = v0 + lane; v < v1; v += 32) {
        float wf[8];
        unpack8(__ldg(wr + v), wf);
#pragma unroll
        for (int t = 0; t < T; ++t) {
          float xf[8];
          unpack8(__ldg(reinterpret_cast<const uint4*>(x + (size_t)t * k) + v), xf);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[t] = fmaf(wf[j], xf[j], acc[t]);
        }
      }
    }
#pragma unroll
    for (int t = 0; t < T; ++t) {
      float a = acc[t];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
      if (lane == 0 && row < n) partial[((size_t)ks * kMaxTokens + t) * kMaxN + row] = a;
    }
  }
  // the block that arrives last for this row block adds the splits in order and writes the output
  __threadfence();
  __syncthreads();
  __shared__ int is_last;
  if (threadIdx.x == 0) is_last = (atomicAdd(&counters[blockIdx.x], 1u) == (unsigned)(splits - 1));
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int e = threadIdx.x; e < kRowsPerBlock * T; e += blockDim.x) {
    const int t = e / kRowsPerBlock, row = blockIdx.x * kRowsPerBlock + e % kRowsPerBlock;
    if (row >= n) continue;
    float s = 0.f;
    for (int q = 0; q < splits; ++q) s += __ldcg(&partial[((size_t)q * kMaxTokens + t) * kMaxN + row]);
    if (res != nullptr) s += __bfloat162float(res[(size_t)t * n + row]);
    out[(size_t)t * n + row] = __float2bfloat16_rn(s);
  }
  if (threadIdx.x == 0) counters[blockIdx.x] = 0u;
}

// Device address of g_scratch on the current device, resolved on first use there.
int scratch_for_current_device(unsigned char** out) {
  static unsigned char* per_device[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    fprintf(stderr, "mk_linear_static: cudaGetDevice failed: %s\n", cudaGetErrorString(e));
    return MK_E_CUDA;
  }
  if (per_device[dev] == nullptr) {
    unsigned char* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_scratch);
    if (e != cudaSuccess || p == nullptr) {
      fprintf(stderr, "mk_linear_static: cudaGetSymbolAddress failed on device %d: %s\n", dev, cudaGetErrorString(e));
      return MK_E_CUDA;
    }
    per_device[dev] = p;
  }
  *out = per_device[dev];
  return 0;
}

}  // namespace

extern "C" int mk_linear_static(const void* x, const void* w, const void* residual, void* out, int tokens, int n, int k,
                                void* stream) {
  if (!x || !w || !out) {
    fprintf(stderr, "mk_linear_static: x, w and out must be device pointers\n");
    return MK_E_INVALID;
  }
  if (tokens < 1 || n < 1 || k < 8 || (k & 7)) {
    fprintf(stderr, "mk_linear_static: need tokens >= 1, n >= 1 and k a positive multiple of 8 (got %d, %d, %d)\n", tokens, n, k);
    return MK_E_INVALID;
  }
  if (tokens > kMaxTokens || n > kMaxN || k > kMaxK) {
    fprintf(stderr,
            "mk_linear_static: %d tokens x %d outputs x %d inputs exceeds the built-in scratch (at most %d x %d x %d); "
            "use the PersistentKernel path for larger layers\n",
            tokens, n, k, kMaxTokens, kMaxN, kMaxK);
    return MK_E_TOO_LARGE;
  }
  if ((((uintptr_t)x) | ((uintptr_t)w) | ((uintptr_t)out)) & 15) {
    fprintf(stderr, "mk_linear_static: pointers must be 16-byte aligned\n");
    return MK_E_INVALID;
  }
  unsigned char* scratch = nullptr;
  if (int rc = scratch_for_current_device(&scratch)) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(scratch, 0, kCounterBytes, s);  // the arrival counters start at zero
  if (e != cudaSuccess) {
    fprintf(stderr, "mk_linear_static: clearing the counters failed: %s\n", cudaGetErrorString(e));
    return MK_E_CUDA;
  }
  int splits = (k + 1023) / 1024;
  splits = splits < 1 ? 1 : (splits > kMaxSplits ? kMaxSplits : splits);
  dim3 grid((n + kRowsPerBlock - 1) / kRowsPerBlock, splits);
  const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
  const __nv_bfloat16* wb = (const __nv_bfloat16*)w;
  const __nv_bfloat16* rb = (const __nv_bfloat16*)residual;
  __nv_bfloat16* ob = (__nv_bfloat16*)out;
  switch (tokens) {
    case 1: linear_static_kernel<1><<<grid, 256, 0, s>>>(xb, wb, rb, ob, n, k, splits, scratch); break;
    case 2: linear_static_kernel<2><<<grid, 256, 0, s>>>(xb, wb, rb, ob, n, k, splits, scratch); break;
    case 3: linear_static_kernel<3><<<grid, 256, 0, s>>>(xb, wb, rb, ob, n, k, splits, scratch); break;
    case 4: linear_static_kernel<4><<<grid, 256, 0, s>>>(xb, wb, rb, ob, n, k, splits, scratch); break;
    case 5: linear_static_kernel<5><<<grid, 256, 0, s>>>(xb, wb, rb, ob, n, k, splits, scratch); break;
    case 6: linear_static_kernel<6><<<grid, 256, 0, s>>>(xb, wb, rb, ob, n, k, splits, scratch); break;
    case 7: linear_static_kernel<7><<<grid, 256, 0, s>>>(xb, wb, rb, ob, n, k, splits, scratch); break;
    default: linear_static_kernel<8><<<grid, 256, 0, s>>>(xb, wb, rb, ob, n, k, splits, scratch); break;
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    fprintf(stderr, "mk_linear_static: launch failed: %s\n", cudaGetErrorString(e));
    return MK_E_CUDA;
  }
  return 0;
}
