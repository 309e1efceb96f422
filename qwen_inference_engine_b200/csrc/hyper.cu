// hyper.cu -- hyper-connections: a model that carries `streams` copies of the residual stream.  A sublayer reads a
// learned combination of the streams (then the RMS norm), and writes back by mixing the streams with a learned matrix
// and adding its output with a learned factor per stream.  One kernel does a sublayer's write and the next sublayer's
// read + norm, one CTA per row; all arithmetic is fp32 and every reduction has a fixed order per row.
#include "fosavik.h"
#include "launch.h"

namespace qie {
namespace {

constexpr int HC_MAX_STREAMS = 8;

__device__ __forceinline__ float block_sum_hc(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = l < nw ? red[l] : 0.f;
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

__global__ void embed_streams_kernel(float* __restrict__ X, const bf16* __restrict__ embed, const bf16* __restrict__ pos_table,
                                     const int* __restrict__ ids, const int* __restrict__ pos, int width, int streams) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const bf16* src = embed + (size_t)ids[r] * width;
  const bf16* pp = pos_table ? pos_table + (size_t)pos[r] * width : nullptr;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = bf2f(src[i]) + (pp ? bf2f(pp[i]) : 0.f);
    for (int s = 0; s < streams; ++s) X[((size_t)r * streams + s) * width + i] = v;
  }
}

template <int S>
__global__ void __launch_bounds__(256) hyper_step_kernel(const HyperStep a) {
  __shared__ float red[32];
  __shared__ float mix[S * S], outv[S], inv[S];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const int W = a.width;
  if (threadIdx.x < S * S && a.y1) mix[threadIdx.x] = bf2f(a.mix[threadIdx.x]);
  if (threadIdx.x < S) {
    if (a.y1) outv[threadIdx.x] = bf2f(a.out[threadIdx.x]);
    inv[threadIdx.x] = a.in ? bf2f(a.in[threadIdx.x]) : 1.0f;
  }
  __syncthreads();
  const int src = a.gather ? a.gather[r] : r;  // the write half is never combined with a gather
  float* Xr = a.X + (size_t)src * S * W;
  float sq = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float x[S];
#pragma unroll
    for (int s = 0; s < S; ++s) x[s] = Xr[(size_t)s * W + i];
    if (a.y1) {
      float yv = a.s1 * a.y1[(size_t)r * W + i];
      if (a.y2) yv = fmaf(a.s2, a.y2[(size_t)r * W + i], yv);
      float nx[S];
#pragma unroll
      for (int t = 0; t < S; ++t) {
        float v = outv[t] * yv;
#pragma unroll
        for (int s = 0; s < S; ++s) v = fmaf(mix[s * S + t], x[s], v);
        nx[t] = v;
      }
#pragma unroll
      for (int t = 0; t < S; ++t) {
        x[t] = nx[t];
        Xr[(size_t)t * W + i] = nx[t];
      }
    }
    if (a.h || a.sum_out) {
      float u = 0.f;
#pragma unroll
      for (int s = 0; s < S; ++s) u = fmaf(inv[s], x[s], u);
      sq = fmaf(u, u, sq);
      if (a.sum_out) a.sum_out[(size_t)r * W + i] = u;
      if (a.h) a.h[(size_t)r * W + i] = u;  // normed below
    }
  }
  if (!a.h || !a.w) return;
  const float rstd = 1.0f / sqrtf(block_sum_hc(sq, red) / (float)W + a.eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) a.h[(size_t)r * W + i] = a.h[(size_t)r * W + i] * rstd * bf2f(a.w[i]);
}

}  // namespace

cudaError_t launch_embed_streams(float* X, const bf16* embed, const bf16* pos_table, const int* ids, const int* pos, int width, int streams,
                                 int n, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  return launch_k(embed_streams_kernel, dim3(n), dim3(width >= 1024 ? 256 : 128), 0, st, X, embed, pos_table, ids, pos, width, streams);
}

cudaError_t launch_hyper_step(const HyperStep& a, cudaStream_t st) {
  if (a.n <= 0) return cudaSuccess;
  if (a.streams < 1 || a.streams > HC_MAX_STREAMS) return cudaErrorInvalidValue;
  if (a.y1 && a.gather) return cudaErrorInvalidValue;
  const dim3 grid(a.n), block(256);
  switch (a.streams) {
    case 1: return launch_k(hyper_step_kernel<1>, grid, block, 0, st, a);
    case 2: return launch_k(hyper_step_kernel<2>, grid, block, 0, st, a);
    case 3: return launch_k(hyper_step_kernel<3>, grid, block, 0, st, a);
    case 4: return launch_k(hyper_step_kernel<4>, grid, block, 0, st, a);
    case 5: return launch_k(hyper_step_kernel<5>, grid, block, 0, st, a);
    case 6: return launch_k(hyper_step_kernel<6>, grid, block, 0, st, a);
    case 7: return launch_k(hyper_step_kernel<7>, grid, block, 0, st, a);
    default: return launch_k(hyper_step_kernel<8>, grid, block, 0, st, a);
  }
}

}  // namespace qie
