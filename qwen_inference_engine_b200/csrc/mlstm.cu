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
  const int nblk = (vd + 31) / 32;  // copies of n and m (mlstm_state_floats); this kernel keeps copy 0
  float* ng = st + (size_t)H * d * vd + (size_t)h * nblk * d;
  float* mg = st + (size_t)H * d * vd + (size_t)H * nblk * d + (size_t)h * nblk;
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


// The same recurrence with the state in registers: a CTA owns 32 columns of one head's S for one segment, warp w
// the rows [w * DPT, (w + 1) * DPT) of them (dim <= 4 * DPT), so a token costs DPT fused multiply-adds per thread, one
// shared-memory reduction over the 4 warps (one barrier) and no global-memory latency: the inputs of the next 16
// tokens (q, k, this CTA's v columns, the log gates) are fetched into registers while the current 16 are computed from
// shared memory.  n and m are kept by every CTA of the head (the same arithmetic, own copy), the
// raw outputs S^T q / denominator go to `out`; the per-head unit norm, norm weight and output gate follow in
// mlstm_out_kernel because they need all columns of the head.
template <int DPT>
__global__ void __launch_bounds__(288) mlstm_scan_reg_kernel(const MlstmArgs a) {
  constexpr int CH = 16, NW = 8, NT = NW * 32;  // tokens staged per chunk; compute warps (a ninth warp finishes tokens)  // tokens staged per chunk
  // [2][CH][stride]: q (scaled, zero-padded to 4 * DPT) | k (same) | v of this CTA's 32 columns | log input gate | log forget gate
  extern __shared__ float4 s_in4[];
  float* s_in = reinterpret_cast<float*>(s_in4);
  __shared__ float s_part[2][NW][32];
  __shared__ float s_dot[2][NW];
  pdl_wait();
  pdl_trigger();
  const int d = a.dim, vd = a.vdim, H = a.heads;
  const int seg = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
  const int col0 = blockIdx.z * 32, col = col0 + lane;
  const bool col_ok = col < vd;
  const int r0 = a.seg_start[seg], r1 = a.seg_start[seg + 1];
  if (r0 >= r1) return;
  float* st = a.state + (size_t)a.seg_slot[seg] * a.slot_stride;
  float* Sg = st + (size_t)h * d * vd;
  // every column block keeps its own copy of n and m: the CTAs of a head run independently, none reads what another writes
  const int nblk = gridDim.z;
  float* ng = st + (size_t)H * d * vd + ((size_t)h * nblk + blockIdx.z) * d;
  float* mg = st + (size_t)H * d * vd + (size_t)H * nblk * d + (size_t)h * nblk + blockIdx.z;
  const bool outw = w == NW;  // the last warp only finishes tokens: sums the partial results, divides, stores
  const int i0 = outw ? d : w * DPT;
  float S[DPT], nn[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    const bool ok = i0 + i < d;
    S[i] = ok && col_ok ? Sg[(size_t)(i0 + i) * vd + col] : 0.f;
    nn[i] = ok ? ng[i0 + i] : 0.f;
  }
  float m = *mg;
  const float qs = rsqrtf((float)d);
  const int ld = a.ld;
  constexpr int DQ = NW * DPT, stride = 2 * DQ + 36;  // a multiple of 4 floats: rows are read with 16-byte loads
  constexpr int PER = (stride + NT - 1) / NT;       // staged elements of one token per thread
  float stage[CH][PER];
  // the inputs of chunk c: global -> registers (in flight while the previous chunk is computed) -> shared memory
  auto fetch = [&](int c) {
#pragma unroll
    for (int t = 0; t < CH; ++t) {
      const int r = r0 + c * CH + t;
      const float* row = a.qkvg + (size_t)min(r, r1 - 1) * ld;
#pragma unroll
      for (int u = 0; u < PER; ++u) {
        const int j = tid + u * NT;
        float v = 0.f;
        if (j < DQ) v = j < d ? row[h * d + j] * qs : 0.f;
        else if (j < 2 * DQ) v = j - DQ < d ? row[H * d + h * d + (j - DQ)] : 0.f;
        else if (j < 2 * DQ + 32) v = col0 + j - 2 * DQ < vd ? row[2 * H * d + h * vd + col0 + j - 2 * DQ] : 0.f;
        else if (j == 2 * DQ + 32) v = a.gates[(size_t)min(r, r1 - 1) * 2 * H + h];       // log gates, transformed by mlstm_gates_kernel
        else if (j == 2 * DQ + 33) v = a.gates[(size_t)min(r, r1 - 1) * 2 * H + H + h];
        stage[t][u] = v;
      }
    }
  };
  auto put = [&](int c) {
    float* dst = s_in + (size_t)(c & 1) * CH * stride;
#pragma unroll
    for (int t = 0; t < CH; ++t)
#pragma unroll
      for (int u = 0; u < PER; ++u) {
        const int j = tid + u * NT;
        if (j < stride) dst[t * stride + j] = stage[t][u];
      }
  };
  const int n_chunks = (r1 - r0 + CH - 1) / CH;
  if (!outw) {
    fetch(0);
    put(0);
  }
  __syncthreads();
  int par = 0;
  for (int c = 0; c < n_chunks; ++c) {
    if (c + 1 < n_chunks && !outw) fetch(c + 1);
    const float* in = s_in + (size_t)(c & 1) * CH * stride;
    const int nt = min(CH, r1 - r0 - c * CH);
    for (int t = 0; t < nt; ++t) {
      const float* tk = in + t * stride;
      const float ig = tk[2 * DQ + 32], fg = tk[2 * DQ + 33];
      const float m_new = fmaxf(fg + m, ig);
      if (!outw) {
        const float v = tk[2 * DQ + lane];
        const float4* q4 = reinterpret_cast<const float4*>(tk + i0);
        const float4* k4 = reinterpret_cast<const float4*>(tk + DQ + i0);
        const float ea = expf(fg + m - m_new), eb = expf(ig - m_new);
        const float bv = eb * v;
        float acc = 0.f, dpart = 0.f;
#pragma unroll
        for (int i4 = 0; i4 < DPT / 4; ++i4) {
          const float4 qv = q4[i4], kv = k4[i4];
          const float q[4] = {qv.x, qv.y, qv.z, qv.w}, k[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int i = i4 * 4 + u;
            S[i] = fmaf(ea, S[i], k[u] * bv);
            acc = fmaf(S[i], q[u], acc);
            nn[i] = fmaf(ea, nn[i], eb * k[u]);
            dpart = fmaf(nn[i], q[u], dpart);  // the same in every lane of the warp
          }
        }
        s_part[par][w][lane] = acc;
        if (lane == 0) s_dot[par][w] = dpart;
      }
      __syncthreads();  // one barrier per token: the partial sums alternate between two buffers
      if (outw) {
        float dot = 0.f, num = 0.f;
#pragma unroll
        for (int x = 0; x < NW; ++x) dot += s_dot[par][x], num += s_part[par][x][lane];
        const float den = fmaxf(fabsf(dot), expf(-m_new)) + 1e-6f;
        const float o = num / den;
        if (col_ok) a.out[(size_t)(r0 + c * CH + t) * H * vd + h * vd + col] = o;
      }
      par ^= 1;
      m = m_new;
    }
    if (c + 1 < n_chunks && !outw) put(c + 1);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    if (i0 + i < d) {
      if (col_ok) Sg[(size_t)(i0 + i) * vd + col] = S[i];
      if (lane == 0) ng[i0 + i] = nn[i];
    }
  }
  if (tid == 0) *mg = m;
}

// pre-activations -> log gates, in place, for all rows at once (tanh, log-sigmoid and exp cost a few hundred instructions
// per value: inside the scan they were the critical path of every token)
__global__ void mlstm_gates_kernel(float* gates, int n, int H, float cap) {
  pdl_wait();
  pdl_trigger();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n * 2 * H) return;
  const float z = cap * tanhf(gates[i] / cap);
  gates[i] = (i % (2 * H)) < H ? z : log_sigmoid(z);
}

// grid (rows, heads): out = rms_unit(out) * w_norm * sigmoid(gate), in place
__global__ void mlstm_out_kernel(const MlstmArgs a) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, h = blockIdx.y, vd = a.vdim, H = a.heads;
  float* o = a.out + (size_t)r * H * vd + h * vd;
  const float* g = a.qkvg + (size_t)r * a.ld + 2 * H * a.dim + H * vd + h * vd;
  float sq = 0.f;
  for (int j = threadIdx.x; j < vd; j += blockDim.x) sq = fmaf(o[j], o[j], sq);
  const float rinv = 1.0f / sqrtf(block_sum_m(sq, red) / (float)vd + a.eps);
  for (int j = threadIdx.x; j < vd; j += blockDim.x) o[j] = o[j] * rinv * bf2f(a.w_norm[h * vd + j]) / (1.0f + expf(-g[j]));
}

}  // namespace

cudaError_t launch_mlstm_scan(const MlstmArgs& a, cudaStream_t st) {
  if (a.n_seg <= 0) return cudaSuccess;
  if (a.dim <= 128) {  // state in registers, 32 columns per CTA
    const dim3 grid(a.n_seg, a.heads, (a.vdim + 31) / 32);
    cudaError_t rg = launch_k(mlstm_gates_kernel, dim3((a.n_rows * 2 * a.heads + 255) / 256), dim3(256), 0, st, a.gates, a.n_rows, a.heads, a.gate_cap);
    if (rg != cudaSuccess) return rg;
    const int dpt = a.dim <= 32 ? 4 : a.dim <= 64 ? 8 : 16;  // rows of S per thread: 8 compute warps split dim
    const size_t smem = (size_t)2 * 16 * (16 * dpt + 36) * sizeof(float);  // two chunks of 16 staged tokens (<= 37 KB)
    cudaError_t r;
    if (a.dim <= 32) r = launch_k(mlstm_scan_reg_kernel<4>, grid, dim3(288), smem, st, a);
    else if (a.dim <= 64) r = launch_k(mlstm_scan_reg_kernel<8>, grid, dim3(288), smem, st, a);
    else r = launch_k(mlstm_scan_reg_kernel<16>, grid, dim3(288), smem, st, a);
    if (r != cudaSuccess) return r;
    return launch_k(mlstm_out_kernel, dim3(a.n_rows, a.heads), dim3(128), 0, st, a);
  }
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
