// attn_gqa.cu -- grouped-query attention over paged key/value rows for the fp32-stream families (fosavik.h): the
// store of new rows (optional per-head unit norm of queries and keys), and an attention whose mask, sink, number of
// score maps and finishing step are arguments: causal or sliding window with kept first tokens, a unit sink in the
// denominator, one or two softmax maps over shared values, and as the last step nothing, a sigmoid gate per head, or
// the differential combination with a unit norm per head.  Softmax and accumulation are fp32; the cache rows are fp32
// or bf16.  Keys are ALWAYS read from the cache (a row's own position is stored first), so a result does not depend
// on how a prompt was cut or what else is in the batch.
#include <algorithm>

#include "fosavik.h"
#include "launch.h"

namespace qie {
namespace {

constexpr int ATK = 32;       // keys per tile
constexpr int ATHREADS = 128;
constexpr int AMAXACC = 16;   // accumulators per thread: query vectors x value columns of a CTA <= 2048

__device__ __forceinline__ const char* kv_row_ptr(const KvRowCache& c, const int* block_table, int max_pages, int slot, int pos) {
  const int page = block_table[(size_t)slot * max_pages + pos / c.page_size];
  const size_t off = (size_t)page * c.page_elems + c.layer_off + (size_t)(pos % c.page_size) * (c.kw + c.vw);
  return static_cast<const char*>(c.pool) + off * c.elt_bytes;
}

__device__ __forceinline__ void store_elt(const KvRowCache& c, char* row, int i, float v) {
  if (c.elt_bytes == 4) reinterpret_cast<float*>(row)[i] = v;
  else reinterpret_cast<bf16*>(row)[i] = f2bf(v);
}

// one CTA per row, one warp per normed group
__global__ void __launch_bounds__(128) kv_store_rows_kernel(const KvStoreArgs a) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (a.c.pool && a.k) {
    char* row = const_cast<char*>(kv_row_ptr(a.c, a.block_table, a.max_pages, a.slot[r], a.pos[r]));
    const float* k = a.k + (size_t)r * a.ldk;
    if (a.k_norm) {
      const int d = a.norm_dim;
      for (int g = warp; g < a.c.kw / d; g += nw) {
        float s = 0.f;
        for (int i = lane; i < d; i += 32) s = fmaf(k[g * d + i], k[g * d + i], s);
        const float rstd = 1.0f / sqrtf(warp_sum(s) / (float)d + a.eps);
        for (int i = lane; i < d; i += 32) store_elt(a.c, row, g * d + i, k[g * d + i] * rstd * bf2f(a.k_norm[i]));
      }
    } else {
      for (int i = threadIdx.x; i < a.c.kw; i += blockDim.x) store_elt(a.c, row, i, k[i]);
    }
    const float* v = a.v + (size_t)r * a.ldv;
    for (int i = threadIdx.x; i < a.c.vw; i += blockDim.x) store_elt(a.c, row, a.c.kw + i, v[i]);
  }
  if (a.q && a.q_norm) {
    float* q = a.q + (size_t)r * a.ldq;
    const int d = a.norm_dim;
    for (int h = warp; h < a.q_heads; h += nw) {
      float s = 0.f;
      for (int i = lane; i < d; i += 32) s = fmaf(q[h * d + i], q[h * d + i], s);
      const float rstd = 1.0f / sqrtf(warp_sum(s) / (float)d + a.eps);
      for (int i = lane; i < d; i += 32) q[h * d + i] = q[h * d + i] * rstd * bf2f(a.q_norm[i]);
    }
  }
}

// CTA (row, kv head x head chunk, key split).  Shared memory: q [QV][dim] (scaled) | K tile [ATK][kd + 1] | V tile
// [ATK][vd] | scores [QV][ATK] | corr [QV] | m [QV] | l [QV], QV = hpc * maps query vectors, kd = maps * dim.
__global__ void __launch_bounds__(ATHREADS) gqa_attention_kernel(const GqaAttnArgs a, int hpc, int chunks, int n_splits) {
  extern __shared__ float sm[];
  __shared__ const char* rowp[ATK];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, split = blockIdx.z;
  const int g = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
  const int hpg = a.heads / a.kv_heads;
  const int h0 = g * hpg + chunk * hpc;                 // first head of this CTA
  const int nh = min(hpc, hpg - chunk * hpc);           // heads of this CTA
  const int maps = a.maps, dim = a.dim, vd = a.vdim, kd = maps * dim;
  const int QV = nh * maps;
  float* qs = sm;
  float* Kt = qs + hpc * maps * dim;
  float* Vt = Kt + ATK * (kd + 1);
  float* sc = Vt + ATK * vd;
  float* corr = sc + hpc * maps * ATK;
  float* mrun = corr + hpc * maps;
  float* lrun = mrun + hpc * maps;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int pos = a.pos[r], slot = a.slot[r];
  // visible keys as one virtual range: the kept first tokens below the window, then the window
  const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  const int nfirst = a.window > 0 ? min(a.keep_first, lo) : 0;
  const int nkeys = nfirst + (pos - lo + 1);
  int per = (nkeys + n_splits - 1) / n_splits;
  per = (per + ATK - 1) / ATK * ATK;
  const int i0 = split * per, i1 = min(nkeys, i0 + per);
  {
    const float* q = a.q + (size_t)r * a.ldq + (size_t)h0 * kd;
    for (int i = tid; i < QV * dim; i += ATHREADS) qs[i] = q[i] * a.scale;
    for (int i = tid; i < QV; i += ATHREADS) mrun[i] = -INFINITY, lrun[i] = 0.f;
  }
  float acc[AMAXACC];
#pragma unroll
  for (int i = 0; i < AMAXACC; ++i) acc[i] = 0.f;
  const int nacc = QV * vd;
  const size_t koff = (size_t)g * kd, voff = (size_t)a.c.kw + (size_t)g * vd;
  for (int t0 = i0; t0 < i1; t0 += ATK) {
    const int nk = min(ATK, i1 - t0);
    __syncthreads();  // the previous tile is consumed; q and m/l are written
    if (tid < nk) {
      const int i = t0 + tid;
      const int j = i < nfirst ? i : lo + (i - nfirst);
      rowp[tid] = kv_row_ptr(a.c, a.block_table, a.max_pages, slot, j);
    }
    __syncthreads();
    if (a.c.elt_bytes == 4) {
      for (int i = tid; i < nk * kd; i += ATHREADS) {
        const int key = i / kd, c = i - key * kd;
        Kt[key * (kd + 1) + c] = reinterpret_cast<const float*>(rowp[key])[koff + c];
      }
      for (int i = tid; i < nk * vd; i += ATHREADS) {
        const int key = i / vd, c = i - key * vd;
        Vt[key * vd + c] = reinterpret_cast<const float*>(rowp[key])[voff + c];
      }
    } else {
      for (int i = tid; i < nk * kd; i += ATHREADS) {
        const int key = i / kd, c = i - key * kd;
        Kt[key * (kd + 1) + c] = bf2f(reinterpret_cast<const bf16*>(rowp[key])[koff + c]);
      }
      for (int i = tid; i < nk * vd; i += ATHREADS) {
        const int key = i / vd, c = i - key * vd;
        Vt[key * vd + c] = bf2f(reinterpret_cast<const bf16*>(rowp[key])[voff + c]);
      }
    }
    __syncthreads();
    // scores: (query vector, key) pairs, key fastest
    for (int i = tid; i < QV * ATK; i += ATHREADS) {
      const int qv = i / ATK, key = i - qv * ATK;
      float s = -INFINITY;
      if (key < nk) {
        const float* qp = qs + qv * dim;
        const float* kp = Kt + key * (kd + 1) + (qv % maps) * dim;
        s = 0.f;
        for (int c = 0; c < dim; ++c) s = fmaf(qp[c], kp[c], s);
      }
      sc[i] = s;
    }
    __syncthreads();
    // online softmax per query vector: a warp per vector, a lane per key
    for (int qv = warp; qv < QV; qv += ATHREADS / 32) {
      const float s = sc[qv * ATK + lane];
      const float mo = mrun[qv];
      const float mn = fmaxf(mo, warp_max(s));
      float p = 0.f, cf = 1.f;
      if (mn > -INFINITY) {
        cf = expf(mo - mn);  // mo = -inf: 0
        p = expf(s - mn);
      }
      const float ps = warp_sum(p);
      sc[qv * ATK + lane] = p;
      if (lane == 0) {
        corr[qv] = cf;
        mrun[qv] = mn;
        lrun[qv] = lrun[qv] * cf + ps;
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < AMAXACC; ++i) {
      const int idx = tid + i * ATHREADS;
      if (idx < nacc) {
        const int qv = idx / vd, col = idx - qv * vd;
        float v = acc[i] * corr[qv];
        const float* pp = sc + qv * ATK;
        for (int key = 0; key < nk; ++key) v = fmaf(pp[key], Vt[key * vd + col], v);
        acc[i] = v;
      }
    }
  }
  __syncthreads();
  // partial (m, l, acc) of (row, head, map, split)
#pragma unroll
  for (int i = 0; i < AMAXACC; ++i) {
    const int idx = tid + i * ATHREADS;
    if (idx < nacc) {
      const int qv = idx / vd, col = idx - qv * vd;
      const size_t rec = (((size_t)r * a.heads + h0) * maps + qv) * n_splits + split;
      a.ws[rec * (vd + 2) + 2 + col] = acc[i];
    }
  }
  for (int qv = tid; qv < QV; qv += ATHREADS) {
    const size_t rec = (((size_t)r * a.heads + h0) * maps + qv) * n_splits + split;
    a.ws[rec * (vd + 2)] = mrun[qv];
    a.ws[rec * (vd + 2) + 1] = lrun[qv];
  }
}

// CTA (row, head): merges the key splits of each map, adds the sink, applies the finishing step
__global__ void __launch_bounds__(128) gqa_finish_kernel(const GqaAttnArgs a, int n_splits) {
  extern __shared__ float o[];  // [vd]
  __shared__ float red[4];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, h = blockIdx.y, vd = a.vdim, maps = a.maps;
  float wsp[2][16];  // per map and split: weight of the split's accumulator (n_splits <= 16)
  float inv_l[2];
  for (int m = 0; m < maps; ++m) {
    const float* rec = a.ws + ((((size_t)r * a.heads + h) * maps + m) * n_splits) * (vd + 2);
    float M = a.unit_sink ? 0.f : -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, rec[(size_t)s * (vd + 2)]);
    float L = a.unit_sink ? expf(-M) : 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = rec[(size_t)s * (vd + 2)];
      const float w = ms > -INFINITY ? expf(ms - M) : 0.f;
      wsp[m][s] = w;
      L = fmaf(rec[(size_t)s * (vd + 2) + 1], w, L);
    }
    inv_l[m] = 1.0f / L;
  }
  float gate = 1.f;
  if (a.finish == 1) gate = 1.0f / (1.0f + expf(-a.gate[(size_t)r * a.ldg + h]));
  float sq = 0.f;
  for (int c = threadIdx.x; c < vd; c += blockDim.x) {
    float am[2] = {0.f, 0.f};
    for (int m = 0; m < maps; ++m) {
      const float* rec = a.ws + ((((size_t)r * a.heads + h) * maps + m) * n_splits) * (vd + 2);
      float v = 0.f;
      for (int s = 0; s < n_splits; ++s) v = fmaf(rec[(size_t)s * (vd + 2) + 2 + c], wsp[m][s], v);
      am[m] = v * inv_l[m];
    }
    float v = am[0];
    if (a.finish == 1) v *= gate;
    else if (a.finish == 2) v = am[0] - a.lam * am[1];
    o[c] = v;
    sq = fmaf(v, v, sq);
  }
  float rstd = 1.f;
  if (a.finish == 2) {
    sq = warp_sum(sq);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
    rstd = a.post / sqrtf(t / (float)vd + a.eps);
  }
  float* out = a.out + (size_t)r * a.ldo + (size_t)h * vd;
  for (int c = threadIdx.x; c < vd; c += blockDim.x) out[c] = o[c] * rstd;
}

}  // namespace

cudaError_t launch_kv_store_rows(const KvStoreArgs& a, cudaStream_t st) {
  if (a.n <= 0) return cudaSuccess;
  if (a.k_norm && (a.norm_dim <= 0 || a.c.kw % a.norm_dim)) return cudaErrorInvalidValue;
  return launch_k(kv_store_rows_kernel, dim3(a.n), dim3(128), 0, st, a);
}

cudaError_t launch_gqa_attention(const GqaAttnArgs& a, cudaStream_t st, int* n_launches) {
  if (n_launches) *n_launches = 0;
  if (a.n <= 0) return cudaSuccess;
  if (a.maps < 1 || a.maps > 2 || a.heads % a.kv_heads || (a.finish == 2 && a.maps != 2) || a.maps * a.vdim > ATHREADS * AMAXACC)
    return cudaErrorInvalidValue;
  const int hpg = a.heads / a.kv_heads;
  const int hpc = std::max(1, std::min(hpg, ATHREADS * AMAXACC / (a.maps * a.vdim)));
  const int chunks = (hpg + hpc - 1) / hpc;
  // key splits: fill the machine when there are few rows, within the workspace
  int splits = 1;
  const long ctas = (long)a.n * a.kv_heads * chunks;
  if (ctas < 2L * a.num_sms && a.max_keys > 2 * ATK) {
    splits = (int)std::min<long>((2L * a.num_sms + ctas - 1) / ctas, (a.max_keys + 2 * ATK - 1) / (2 * ATK));
    splits = std::max(1, std::min(splits, 16));
  }
  const size_t one = gqa_ws_floats(a.n, a.heads, a.maps, a.vdim);
  if (one > a.ws_floats) return cudaErrorInvalidValue;
  splits = (int)std::min<size_t>(splits, a.ws_floats / one);
  const int kd = a.maps * a.dim, qvm = hpc * a.maps;
  const size_t smem = ((size_t)qvm * a.dim + (size_t)ATK * (kd + 1) + (size_t)ATK * a.vdim + (size_t)qvm * ATK + 3 * (size_t)qvm) * sizeof(float);
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    cudaError_t r = cudaFuncSetAttribute(gqa_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (r != cudaSuccess) return r;
  }
  cudaError_t r = launch_k(gqa_attention_kernel, dim3(a.n, a.kv_heads * chunks, splits), dim3(ATHREADS), smem, st, a, hpc, chunks, splits);
  if (r != cudaSuccess) return r;
  if (n_launches) *n_launches = 2;
  return launch_k(gqa_finish_kernel, dim3(a.n, a.heads), dim3(128), (size_t)a.vdim * sizeof(float), st, a, splits);
}

}  // namespace qie
