// mlstm.cu -- the matrix-memory recurrence of xLSTM (mLSTM) with a state slot per sequence (nogatar.h).
//
// Per head, with log input gate i_t = cap * tanh(zi / cap), log forget gate f_t = logsigmoid(cap * tanh(zf / cap))
// and a running maximum m (m_0 = 0, S_0 = 0, n_0 = 0):
//   m_t = max(f_t + m_{t-1}, i_t)
//   S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T        (S: [dim, vdim])
//   n_t = exp(f_t + m_{t-1} - m_t) n_{t-1} + exp(i_t - m_t) k_t
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6),   q_t scaled by dim^-1/2
// followed by the per-head unit RMS norm, the norm weight and the sigmoid output gate.  Everything here is
// fp32.  One CTA per (sequence segment, head) walks the segment's rows in order with S in shared memory (or in
// place in global memory when it does not fit) and writes the state back, so a prompt cut into portions, a
// single decoded token and a whole prompt run the same arithmetic in the same order.
#include "launch.h"
#include "nogatar.h"

namespace qie {
namespace {

__device__ __forceinline__ float block_sum_m(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = l < nw ? red[l] : 0.f;
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

__device__ __forceinline__ float log_sigmoid(float x) { return x >= 0.f ? -log1pf(expf(-x)) : x - log1pf(expf(x)); }

__global__ void __launch_bounds__(128) mlstm_scan_kernel(const MlstmArgs a, int s_in_smem) {
  extern __shared__ float sh[];
  pdl_wait();
  pdl_trigger();
  const int d = a.dim, vd = a.vdim, H = a.heads;
  float* s_q = sh;
  float* s_k = s_q + d;
  float* s_n = s_k + d;
  float* s_o = s_n + d;
  float* red = s_o + vd;
  float* s_S = red + 32;
  const int seg = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, nt = blockDim.x;
  const int r0 = a.seg_start[seg], r1 = a.seg_start[seg + 1];
  float* st = a.state + (size_t)a.seg_slot[seg] * a.slot_stride;
  float* Sg = st + (size_t)h * d * vd;
  float* ng = st + (size_t)H * d * vd + (size_t)h * d;
  float* mg = st + (size_t)H * d * vd + (size_t)H * d + h;
  float* S = s_in_smem ? s_S : Sg;
  if (s_in_smem)
    for (int i = tid; i < d * vd; i += nt) s_S[i] = Sg[i];
  for (int i = tid; i < d; i += nt) s_n[i] = ng[i];
  float m = *mg;
  const float qs = rsqrtf((float)d);
  const int ld = a.ld;
  for (int r = r0; r < r1; ++r) {
    const float* row = a.qkvg + (size_t)r * ld;
    const float* v = row + 2 * H * d + h * vd;
    const float* g = row + 2 * H * d + H * vd + h * vd;
    __syncthreads();  // s_q / s_k / s_o of the previous row are no longer read
    for (int i = tid; i < d; i += nt) {
      s_q[i] = row[h * d + i] * qs;
      s_k[i] = row[H * d + h * d + i];
    }
    const float zi = a.gates[(size_t)r * 2 * H + h], zf = a.gates[(size_t)r * 2 * H + H + h];
    const float ig = a.gate_cap * tanhf(zi / a.gate_cap);
    const float fg = log_sigmoid(a.gate_cap * tanhf(zf / a.gate_cap));
    const float m_new = fmaxf(fg + m, ig);
    const float ea = expf(fg + m - m_new), eb = expf(ig - m_new);
    __syncthreads();
    float part = 0.f;
    for (int i = tid; i < d; i += nt) {
      const float nn = ea * s_n[i] + eb * s_k[i];
      s_n[i] = nn;
      part = fmaf(nn, s_q[i], part);
    }
    const float dot = block_sum_m(part, red);
    const float den = fmaxf(fabsf(dot), expf(-m_new)) + 1e-6f;
    float sq = 0.f;
    for (int j = tid; j < vd; j += nt) {
      const float bv = eb * v[j];
      float acc = 0.f;
      for (int i = 0; i < d; ++i) {
        const float s = fmaf(ea, S[(size_t)i * vd + j], s_k[i] * bv);
        S[(size_t)i * vd + j] = s;
        acc = fmaf(s, s_q[i], acc);
      }
      const float o = acc / den;
      s_o[j] = o;
      sq = fmaf(o, o, sq);
    }
    const float rinv = 1.0f / sqrtf(block_sum_m(sq, red) / (float)vd + a.eps);
    for (int j = tid; j < vd; j += nt) {
      const float gate = 1.0f / (1.0f + expf(-g[j]));
      a.out[(size_t)r * H * vd + h * vd + j] = s_o[j] * rinv * bf2f(a.w_norm[h * vd + j]) * gate;
    }
    m = m_new;
  }
  __syncthreads();
  if (s_in_smem)
    for (int i = tid; i < d * vd; i += nt) Sg[i] = s_S[i];
  for (int i = tid; i < d; i += nt) ng[i] = s_n[i];
  if (tid == 0) *mg = m;
}

}  // namespace

cudaError_t launch_mlstm_scan(const MlstmArgs& a, cudaStream_t st) {
  if (a.n_seg <= 0) return cudaSuccess;
  const size_t base = (size_t)(3 * a.dim + a.vdim + 32) * sizeof(float);
  const size_t with_s = base + (size_t)a.dim * a.vdim * sizeof(float);
  const int in_smem = with_s <= 200 * 1024 ? 1 : 0;
  const size_t smem = in_smem ? with_s : base;
  if (smem > 48 * 1024) {
    cudaError_t r = cudaFuncSetAttribute(mlstm_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (r != cudaSuccess) return r;
  }
  return launch_k(mlstm_scan_kernel, dim3(a.n_seg, a.heads), dim3(128), smem, st, a, in_smem);
}

}  // namespace qie
