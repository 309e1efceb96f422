// fosavik_model.cu -- the Fosavik family on the engine: configuration reader (config.json), weight loader
// (model.safetensors -> one device blob), the paged key/value rows and the recurrent state slots, and the launch order
// of one forward over a batch of rows.  A row is (sequence slot, position) exactly as in the other families; rows of
// one sequence are consecutive and in position order, rows of different sequences may be portions of prompts next to
// single decoded tokens.  Every size and constant comes from the configuration.
#include "fosavik.h"

#include <math.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <map>

#include "engine.h"
#include "json_min.h"
#include "launch.h"

namespace qie {
namespace {

#define NEED(cond, msg)      \
  do {                       \
    if (!(cond)) return msg; \
  } while (0)

int as_int(const JsonValue* v, int dflt) { return v && v->is_number() ? (int)llround(v->num) : dflt; }
float as_float(const JsonValue* v, float dflt) { return v && v->is_number() ? (float)v->num : dflt; }
bool present(const JsonValue* v) { return v && v->kind != JsonValue::Null; }

std::string parse_attention(const JsonValue& mx, FvAttn* at, bool two_maps) {
  at->heads = as_int(mx.have("heads"), 0);
  at->kv_heads = as_int(mx.have("kv_heads"), at->heads);
  at->dim = as_int(mx.have("dim"), 0);
  at->vdim = as_int(mx.have("vdim"), at->dim);
  at->maps = two_maps ? 2 : 1;
  NEED(at->heads > 0 && at->kv_heads > 0 && at->dim > 0 && at->vdim > 0, "config.json: attention heads / kv_heads / dim / vdim missing");
  NEED(at->heads % at->kv_heads == 0, "config.json: heads must be a multiple of kv_heads");
  NEED(mx.have("scale") && mx.have("scale")->is_number(), "config.json: attention without scale");
  at->scale = (float)mx.have("scale")->num;
  if (const JsonValue* mk = mx.have("mask"))
    if (present(mk)) {
      at->window = as_int(mk->have("size"), 0);
      at->keep_first = as_int(mk->have("keep_first"), 0);
    }
  return "";
}

std::string parse_config(const JsonValue& root, FvModel* m) {
  NEED(root.kind == JsonValue::Object, "config.json: not an object");
  m->vocab = as_int(root.have("vocab"), 0);
  m->width = as_int(root.have("width"), 0);
  m->streams = as_int(root.have("streams"), 1);
  m->max_positions = as_int(root.have("max_positions"), 0);
  NEED(m->vocab > 0 && m->width > 0, "config.json: vocab / width missing");
  NEED(m->streams >= 1 && m->streams <= 8, "config.json: streams must be 1..8");
  NEED(m->max_positions > 0, "config.json: max_positions missing");
  if (const JsonValue* nm = root.have("norm")) m->eps = as_float(nm->have("eps"), 1e-6f);
  const JsonValue* layers = root.have("layers");
  NEED(layers && layers->kind == JsonValue::Array && !layers->arr.empty(), "config.json: layers missing");
  for (const JsonValue& jl : layers->arr) {
    FvLayer L;
    const JsonValue* type = jl.have("type");
    const JsonValue* mx = jl.have("mixer");
    NEED(type && type->kind == JsonValue::String && mx && mx->kind == JsonValue::Object, "config.json: layer without type / mixer");
    if (type->str == "attention") {
      L.type = 0;
      std::string err = parse_attention(*mx, &L.at, true);
      if (!err.empty()) return err;
      NEED(mx->have("diff") && mx->have("diff")->is_number(), "config.json: attention without diff");
      L.diff = (float)mx->have("diff")->num;
      if (present(mx->have("kv_from"))) {
        L.kv_from = as_int(mx->have("kv_from"), -1);
        L.at.own_kv = false;
      }
    } else if (type->str == "parallel") {
      L.type = 1;
      const JsonValue* lf = mx->have("left");
      const JsonValue* rt = mx->have("right");
      NEED(lf && rt, "config.json: parallel mixer without left / right");
      std::string err = parse_attention(*lf, &L.at, false);
      if (!err.empty()) return err;
      NEED(L.at.vdim == L.at.dim, "config.json: the window attention's values are its keys (vdim must equal dim)");
      L.left_scale = as_float(mx->have("left_scale"), 1.f);
      L.right_scale = as_float(mx->have("right_scale"), 1.f);
      L.lru_width = as_int(rt->have("width"), 0);
      L.lru_blocks = as_int(rt->have("blocks"), 1);
      L.lru_taps = as_int(rt->have("conv"), 0);
      NEED(L.lru_width > 0 && L.lru_blocks > 0 && L.lru_width % L.lru_blocks == 0, "config.json: recurrent width must be a multiple of blocks");
      NEED(L.lru_taps >= 1 && L.lru_taps <= 8, "config.json: convolution taps must be 1..8");
    } else if (type->str == "mamba2") {
      L.type = 2;
      L.m_heads = as_int(mx->have("heads"), 0);
      L.m_P = as_int(mx->have("vdim"), 0);
      L.m_N = as_int(mx->have("state"), 0);
      L.m_groups = as_int(mx->have("groups"), 1);
      L.m_norm_groups = as_int(mx->have("norm_groups"), 1);
      L.m_taps = as_int(mx->have("conv"), 0);
      NEED(L.m_heads > 0 && L.m_P > 0 && L.m_N > 0, "config.json: mamba2 heads / vdim / state missing");
      NEED(L.m_groups > 0 && L.m_heads % L.m_groups == 0, "config.json: mamba2 heads must be a multiple of groups");
      NEED(L.m_norm_groups > 0 && (L.m_heads * L.m_P) % L.m_norm_groups == 0, "config.json: mamba2 inner width must be a multiple of norm_groups");
      NEED(L.m_taps >= 1 && L.m_taps <= 8, "config.json: convolution taps must be 1..8");
      NEED(L.m_N <= 2048, "config.json: mamba2 state too large");
    } else {
      return "config.json: unknown layer type '" + type->str + "'";
    }
    if (const JsonValue* mlp = jl.have("mlp"))
      if (present(mlp)) {
        const JsonValue* kind = mlp->have("kind");
        NEED(!kind || kind->str == "dense", "config.json: unknown mlp kind");
        L.ff = as_int(mlp->have("ff"), 0);
        NEED(L.ff > 0, "config.json: mlp without ff");
        NEED(mlp->have("limit") && mlp->have("limit")->is_number(), "config.json: mlp without limit");
        L.limit = (float)mlp->have("limit")->num;
      }
    m->layers.push_back(L);
  }
  for (size_t i = 0; i < m->layers.size(); ++i) {
    FvLayer& L = m->layers[i];
    if (L.type != 0 || L.at.own_kv) continue;
    NEED(L.kv_from >= 0 && L.kv_from < (int)i, "config.json: kv_from must name an earlier layer");
    const FvLayer& S = m->layers[L.kv_from];
    NEED(S.type == 0 && S.at.own_kv, "config.json: kv_from must name an attention layer with projections of its own");
    NEED(S.at.kv_heads == L.at.kv_heads && S.at.dim == L.at.dim && S.at.vdim == L.at.vdim, "config.json: kv_from layer has other key / value sizes");
  }
  return "";
}

// tensors in blob order; tensors that one GEMM reads as a single matrix are adjacent (no padding between them)
std::vector<TensorSpec> build_layout(const FvModel& m) {
  BlobLayout bl;
  auto pad = [&]() { bl.pad(); };
  auto add = [&](const std::string& name, size_t rows, size_t cols, int kind) { bl.add(name, rows, cols, kind); };
  const size_t W = m.width, S = m.streams;
  pad(), add("embed", m.vocab, W, 0);
  pad(), add("pos", m.max_positions, W, 2);
  for (size_t i = 0; i < m.layers.size(); ++i) {
    const FvLayer& L = m.layers[i];
    const std::string p = "l" + std::to_string(i) + ".";
    const size_t H = L.at.heads, G = L.at.kv_heads, d = L.at.dim, vd = L.at.vdim;
    pad(), add(p + "norm1", W, 0, 1);
    pad(), add(p + "hc1.in", S, 0, 2), add(p + "hc1.out", S, 0, 2), add(p + "hc1.mix", S, S, 2);
    if (L.type == 0) {
      pad(), add(p + "mix.q", H * 2 * d, W, 0);
      if (L.at.own_kv) add(p + "mix.k", G * 2 * d, W, 0), add(p + "mix.v", G * vd, W, 0);
      pad(), add(p + "mix.lq1", d, 0, 2), add(p + "mix.lk1", d, 0, 2), add(p + "mix.lq2", d, 0, 2), add(p + "mix.lk2", d, 0, 2);
      pad(), add(p + "mix.o", W, H * vd, 0);
    } else if (L.type == 1) {
      const size_t R = L.lru_width, B = L.lru_blocks, bw = R / B;
      pad(), add(p + "mix.left.q", H * d, W, 0), add(p + "mix.left.k", G * d, W, 0), add(p + "mix.left.g", H, W, 0);
      add(p + "mix.right.y", R, W, 0), add(p + "mix.right.x", R, W, 0);
      pad(), add(p + "mix.left.q.norm", d, 0, 1);
      pad(), add(p + "mix.left.k.norm", d, 0, 1);
      pad(), add(p + "mix.left.o", W, H * vd, 0);
      pad(), add(p + "mix.right.y.b", R, 0, 2);
      pad(), add(p + "mix.right.x.b", R, 0, 2);
      pad(), add(p + "mix.right.conv", R, L.lru_taps, 0);
      pad(), add(p + "mix.right.conv.b", R, 0, 2);
      pad(), add(p + "mix.right.ra", B * bw, bw, 0);
      pad(), add(p + "mix.right.ra.b", R, 0, 2);
      pad(), add(p + "mix.right.ri", B * bw, bw, 0);
      pad(), add(p + "mix.right.ri.b", R, 0, 2);
      pad(), add(p + "mix.right.lam", R, 0, 2);
      pad(), add(p + "mix.right.o", W, R, 0);
    } else {
      const size_t inner = (size_t)L.m_heads * L.m_P, GN = (size_t)L.m_groups * L.m_N, C = inner + 2 * GN;
      pad(), add(p + "mix.in", 2 * inner + 2 * GN + L.m_heads, W, 0);
      pad(), add(p + "mix.conv", C, L.m_taps, 0);
      pad(), add(p + "mix.conv.b", C, 0, 2);
      pad(), add(p + "mix.dt_bias", L.m_heads, 0, 2);
      pad(), add(p + "mix.A_log", L.m_heads, 0, 2);
      pad(), add(p + "mix.D", L.m_heads, 0, 1);
      pad(), add(p + "mix.norm", inner, 0, 1);
      pad(), add(p + "mix.o", W, inner, 0);
    }
    if (L.ff > 0) {
      pad(), add(p + "norm2", W, 0, 1);
      pad(), add(p + "hc2.in", S, 0, 2), add(p + "hc2.out", S, 0, 2), add(p + "hc2.mix", S, S, 2);
      pad(), add(p + "mlp.gate", L.ff, W, 0), add(p + "mlp.up", L.ff, W, 0);
      pad(), add(p + "mlp.down", W, L.ff, 0);
    }
  }
  pad(), add("final.norm", W, 0, 1);
  pad(), add("head", m.vocab, W, 0);
  return bl.t;
}

float bits_to_float(uint16_t b) {
  const uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

#define CUS(expr)                                                      \
  do {                                                                 \
    cudaError_t _e = (expr);                                           \
    if (_e != cudaSuccess) {                                           \
      *code = QIE_ECUDA;                                               \
      return std::string(#expr) + ": " + cudaGetErrorString(_e);       \
    }                                                                  \
  } while (0)

std::string finish_setup(qie_engine* e, const std::vector<TensorSpec>& t, const std::vector<uint16_t>& blob, int* code) {
  FvModel* m = e->fv;
  const qie_engine_opts& o = e->opts;
  // a sequence cannot grow beyond the learned position vectors, whatever the pool holds
  const int context = std::min(o.context, m->max_positions);
  m->f32 = o.compute_dtype == QIE_DTYPE_F32;
  m->blob_bytes = blob.size() * 2;
  CUS(cudaMalloc(&m->blob, m->blob_bytes));
  CUS(cudaMemcpy(m->blob, blob.data(), m->blob_bytes, cudaMemcpyHostToDevice));
  std::map<std::string, const TensorSpec*> at;
  for (const TensorSpec& s : t) at[s.name] = &s;
  auto P = [&](const std::string& n) -> const bf16* {
    auto it = at.find(n);
    return it == at.end() ? nullptr : m->blob + it->second->off;
  };
  // sum_i a[i] * b[i] of two vectors, in fp32 on the host values
  auto dot = [&](const std::string& a, const std::string& b) {
    const TensorSpec *sa = at[a], *sb = at[b];
    float s = 0.f;
    for (size_t i = 0; i < sa->elems(); ++i) s = fmaf(bits_to_float(blob[sa->off + i]), bits_to_float(blob[sb->off + i]), s);
    return s;
  };
  m->embed = P("embed");
  m->pos_table = P("pos");
  m->final_norm = P("final.norm");
  m->head = P("head");
  e->cfg = qie_config{m->width, 0, (int)m->layers.size(), 0, 0, 0, m->vocab, context};
  size_t page_elems = 0, slot_floats = 0;
  size_t w0 = 1, w1 = 1, w2 = 1, w3 = 1, hmv = 1, maxk = m->width;
  std::vector<int> cache_of(m->layers.size(), -1);
  for (size_t i = 0; i < m->layers.size(); ++i) {
    FvLayer& L = m->layers[i];
    const std::string p = "l" + std::to_string(i) + ".";
    const size_t H = L.at.heads, G = L.at.kv_heads, d = L.at.dim, vd = L.at.vdim;
    L.norm1 = P(p + "norm1");
    L.hc1_in = P(p + "hc1.in"), L.hc1_out = P(p + "hc1.out"), L.hc1_mix = P(p + "hc1.mix");
    if (L.type == 0) {
      L.w_in = P(p + "mix.q");
      L.wo = P(p + "mix.o");
      L.lam = expf(dot(p + "mix.lq1", p + "mix.lk1")) - expf(dot(p + "mix.lq2", p + "mix.lk2")) + L.diff;
      if (L.at.own_kv) {
        cache_of[i] = (int)m->kv_off.size();
        m->kv_off.push_back(page_elems);
        page_elems += (size_t)o.page_size * (G * 2 * d + G * vd);
      } else {
        cache_of[i] = cache_of[L.kv_from];
      }
      L.at.cache_id = cache_of[i];
      w0 = std::max(w0, H * 2 * d + (L.at.own_kv ? G * 2 * d + G * vd : 0));
      w1 = std::max(w1, H * vd);
      hmv = std::max(hmv, H * 2 * (vd + 2));
      maxk = std::max(maxk, H * vd);
    } else if (L.type == 1) {
      const size_t R = L.lru_width;
      L.w_in = P(p + "mix.left.q");
      L.q_norm = P(p + "mix.left.q.norm"), L.k_norm = P(p + "mix.left.k.norm");
      L.wo = P(p + "mix.left.o");
      L.y_b = P(p + "mix.right.y.b"), L.x_b = P(p + "mix.right.x.b");
      L.conv_w = P(p + "mix.right.conv"), L.conv_b = P(p + "mix.right.conv.b");
      L.ra = P(p + "mix.right.ra"), L.ra_b = P(p + "mix.right.ra.b"), L.ri = P(p + "mix.right.ri"), L.ri_b = P(p + "mix.right.ri.b");
      L.lam_w = P(p + "mix.right.lam");
      L.wo2 = P(p + "mix.right.o");
      cache_of[i] = (int)m->kv_off.size();
      L.at.cache_id = cache_of[i];
      m->kv_off.push_back(page_elems);
      page_elems += (size_t)o.page_size * (2 * G * d);
      L.state_off = slot_floats;
      slot_floats += R + (size_t)(L.lru_taps - 1) * R;
      w0 = std::max(w0, H * d + G * d + H + 2 * R);
      w1 = std::max(w1, H * vd);
      w2 = std::max(w2, R);
      w3 = std::max(w3, 2 * R);
      hmv = std::max(hmv, H * (vd + 2));
      maxk = std::max(maxk, std::max(H * vd, R));
    } else {
      const size_t inner = (size_t)L.m_heads * L.m_P, GN = (size_t)L.m_groups * L.m_N, C = inner + 2 * GN;
      L.w_in = P(p + "mix.in");
      L.conv_w = P(p + "mix.conv"), L.conv_b = P(p + "mix.conv.b");
      L.dt_bias = P(p + "mix.dt_bias"), L.A_log = P(p + "mix.A_log"), L.Dw = P(p + "mix.D"), L.gn_w = P(p + "mix.norm");
      L.wo = P(p + "mix.o");
      L.state_off = slot_floats;
      slot_floats += (size_t)L.m_heads * L.m_N * L.m_P + (size_t)(L.m_taps - 1) * C;
      w0 = std::max(w0, 2 * inner + 2 * GN + L.m_heads);
      w1 = std::max(w1, C);
      w2 = std::max(w2, inner);
      w3 = std::max(w3, inner);
      maxk = std::max(maxk, inner);
    }
    if (L.ff > 0) {
      L.norm2 = P(p + "norm2");
      L.hc2_in = P(p + "hc2.in"), L.hc2_out = P(p + "hc2.out"), L.hc2_mix = P(p + "hc2.mix");
      L.w_gu = P(p + "mlp.gate");
      L.w_down = P(p + "mlp.down");
      w0 = std::max(w0, (size_t)2 * L.ff);
      w1 = std::max(w1, (size_t)L.ff);
      maxk = std::max(maxk, (size_t)L.ff);
    }
  }
  // key/value pages (a model without attention layers still counts positions in pages)
  m->page_elems = page_elems;
  const size_t elt = m->f32 ? 4 : 2;
  const size_t page_bytes = std::max<size_t>(page_elems * elt, 16);
  int n_pages = o.max_pages;
  if (n_pages <= 0) n_pages = (int)std::max<size_t>(1, (o.kv_bytes ? o.kv_bytes : ((size_t)1 << 30)) / page_bytes);
  CUS(cudaMalloc(&m->kv_pool, (size_t)n_pages * page_bytes));
  CUS(cudaMemsetAsync(m->kv_pool, 0, (size_t)n_pages * page_bytes, e->stream));
  e->kv = KvGeom{nullptr, n_pages, o.page_size, (int)m->kv_off.size(), 1, 0};
  CUS(engine_alloc_shared(e, n_pages, context));
  // recurrent state slots
  m->slot_floats = slot_floats;
  if (slot_floats) {
    CUS(cudaMalloc(&m->state, (size_t)o.max_seqs * slot_floats * sizeof(float)));
    CUS(cudaMemsetAsync(m->state, 0, (size_t)o.max_seqs * slot_floats * sizeof(float), e->stream));
  }
  // activations
  const size_t R = o.max_batch_tokens, W = m->width;
  auto fbuf = [&](float** p, size_t n) { return cudaMalloc(p, std::max<size_t>(n, 1) * sizeof(float)); };
  CUS(fbuf(&m->X, R * W * m->streams));
  CUS(fbuf(&m->hn, R * W));
  CUS(fbuf(&m->y, R * W));
  CUS(fbuf(&m->y2, R * W));
  CUS(fbuf(&m->p0, R * w0));
  CUS(fbuf(&m->p1, R * w1));
  CUS(fbuf(&m->p2, R * w2));
  CUS(fbuf(&m->p3, R * w3));
  CUS(fbuf(&m->xo, R * W));
  m->attn_ws_floats = (R + 2048) * hmv;  // room for key splits when a step has few rows
  CUS(fbuf(&m->attn_ws, m->attn_ws_floats));
  m->scan_ws_floats = w2 > 1 ? (R / 64 + 64 + 2) * 2 * w2 : 0;
  for (const FvLayer& L : m->layers)
    if (L.type == 2) m->scan_ws_floats = std::max(m->scan_ws_floats, ssd_ws_floats(R, L.m_heads, L.m_N, L.m_P));
  CUS(fbuf(&m->scan_ws, m->scan_ws_floats));
  if (!m->f32) CUS(m->tc.alloc(R, maxk, std::max<size_t>(std::max<size_t>(W, (size_t)m->vocab), w0), e->stream));
  CUS(m->alloc_row_buffers(R));
  e->logits_rows = (int)R;
  CUS(cudaStreamSynchronize(e->stream));
  return "";
}

std::string create_common(qie_engine* e, const std::string& cfg_text, const std::string* st_path, uint64_t seed, int* code) {
  *code = QIE_EIO;
  JsonValue root;
  std::string err;
  if (!JsonReader::parse(cfg_text.data(), cfg_text.data() + cfg_text.size(), &root, &err)) return "config.json: " + err;
  e->fv = new FvModel();
  e->fam = e->fv;
  err = parse_config(root, e->fv);
  if (!err.empty()) return err;
  const std::vector<TensorSpec> t = build_layout(*e->fv);
  std::vector<uint16_t> blob(t.empty() ? 0 : t.back().off + t.back().elems(), 0);
  if (st_path) {
    err = load_safetensors_blob(*st_path, t, &blob);
    if (!err.empty()) return err;
  } else {
    fill_synthetic_blob(t, seed, &blob);
  }
  return finish_setup(e, t, blob, code);
}

}  // namespace

std::string fosavik_create(qie_engine* e, const std::string& dir, int* code) {
  std::string cfg;
  *code = QIE_EIO;
  if (!read_text_file(dir + "/config.json", &cfg)) return "cannot read " + dir + "/config.json";
  const std::string st = dir + "/model.safetensors";
  return create_common(e, cfg, &st, 0, code);
}

std::string fosavik_create_synthetic(qie_engine* e, const std::string& cfg_json, uint64_t seed, int* code) {
  return create_common(e, cfg_json, nullptr, seed, code);
}

void FvModel::release() {
  void* dev[] = {blob, kv_pool, state, X, hn, y, y2, p0, p1, p2, p3, xo, attn_ws, scan_ws};
  tc.release();
  release_row_buffers();
  for (void* p : dev)
    if (p) cudaFree(p);
}

void FvModel::reset_slot(qie_engine* e, int seq) {
  if (state) cudaMemsetAsync(state + (size_t)seq * slot_floats, 0, slot_floats * sizeof(float), e->stream);
}

cudaError_t FvModel::forward(qie_engine* e, int n, int n_seg, int n_out, int max_kv_len, float temperature, bool advance) {
  FvModel* m = this;
  cudaStream_t st = e->stream;
  const int W = m->width, S = m->streams;
  const int rnd = m->f32 ? 0 : 1;  // bf16 serving precision: the operands of the projections are bf16 values
  const int* segs = advance ? m->iota : m->seg_start;
  const int* seg_sl = advance ? e->slot_d : m->seg_slot;
  const int* outs = advance ? m->iota : m->out_rows;
  // plain projection C[n, N] = A[n, K] Wt[N, K]^T: the tcgen05 GEMM when the shape and the precision allow, else the
  // fp32-accumulate kernels (tensor cores on bf16 operands, plain fp32 in 32-bit mode)
  auto proj = [&](const float* A, int lda, const bf16* Wt, int K, int N, float* C, int ldc, int rows) {
    if (!m->f32 && m->tc.fits(rows, K, N, Wt)) return m->tc.gemm(e, A, lda, Wt, K, N, C, ldc, 0, rows);
    GemmF32 g;
    g.A = A, g.lda = lda, g.W = Wt, g.ldw = K, g.C = C, g.ldc = ldc, g.M = rows, g.N = N, g.K = K, g.round_a = rnd;
    return launch_gemm_f32(g, st);
  };
  if (m->dump_layers && !m->layer_dump)
    if (cudaMalloc(&m->layer_dump, m->layers.size() * (size_t)e->opts.max_batch_tokens * W * sizeof(float)) != cudaSuccess) return cudaErrorMemoryAllocation;
  FAM_TRY(KK_EMBED, launch_embed_streams(m->X, m->embed, m->pos_table, e->ids_d, e->pos_d, W, S, n, st));
  {
    HyperStep hs;
    hs.X = m->X, hs.width = W, hs.streams = S, hs.n = n;
    hs.in = m->layers[0].hc1_in, hs.w = m->layers[0].norm1, hs.eps = m->eps, hs.h = m->hn;
    FAM_TRY(KK_HYPER, launch_hyper_step(hs, st));
  }
  for (size_t li = 0; li < m->layers.size(); ++li) {
    const FvLayer& L = m->layers[li];
    const FvAttn& A = L.at;
    const float* y2 = nullptr;
    float s1 = 1.f, s2 = 0.f;
    auto cache_of = [&](const FvAttn& at) {
      KvRowCache c;
      c.pool = m->kv_pool, c.elt_bytes = m->f32 ? 4 : 2, c.page_size = e->kv.page_size, c.page_elems = m->page_elems;
      c.layer_off = m->kv_off[at.cache_id];
      c.kw = at.kv_heads * at.maps * at.dim, c.vw = at.kv_heads * at.vdim;
      return c;
    };
    auto attend = [&](GqaAttnArgs& g) {
      g.c = cache_of(A);
      g.heads = A.heads, g.kv_heads = A.kv_heads, g.dim = A.dim, g.vdim = A.vdim, g.maps = A.maps, g.scale = A.scale;
      g.window = A.window, g.keep_first = A.keep_first, g.eps = m->eps;
      g.pos = e->pos_d, g.slot = e->slot_d, g.block_table = e->block_table_d, g.max_pages = e->max_pages_per_seq, g.n = n, g.max_keys = max_kv_len;
      g.ws = m->attn_ws, g.ws_floats = m->attn_ws_floats, g.num_sms = e->num_sms;
      g.seg_start = segs, g.seg_slot = seg_sl, g.n_seg = n_seg;
      int nl = 0;
      cudaError_t r = launch_gqa_attention(g, st, &nl);
      e->launches += nl > 0 ? nl - 1 : 0;
      return r;
    };
    if (L.type == 0) {
      const int Nq = A.heads * 2 * A.dim, Nk = A.kv_heads * 2 * A.dim, Nv = A.kv_heads * A.vdim;
      const int Nin = Nq + (A.own_kv ? Nk + Nv : 0);
      FAM_TRY(KK_F32_PROJ, proj(m->hn, W, L.w_in, W, Nin, m->p0, Nin, n));
      if (A.own_kv) {
        KvStoreArgs ks;
        ks.c = cache_of(A), ks.k = m->p0 + Nq, ks.ldk = Nin, ks.v = m->p0 + Nq + Nk, ks.ldv = Nin;
        ks.pos = e->pos_d, ks.slot = e->slot_d, ks.block_table = e->block_table_d, ks.max_pages = e->max_pages_per_seq, ks.n = n;
        FAM_TRY(KK_KV_STORE, launch_kv_store_rows(ks, st));
      }
      GqaAttnArgs g;
      g.q = m->p0, g.ldq = Nin, g.out = m->p1, g.ldo = A.heads * A.vdim;
      g.finish = 2, g.lam = L.lam, g.post = 1.0f - L.diff;
      FAM_TRY(KK_GQA_ATTN, attend(g));
      FAM_TRY(KK_F32_PROJ, proj(m->p1, A.heads * A.vdim, L.wo, A.heads * A.vdim, W, m->y, W, n));
    } else if (L.type == 1) {
      const int Nq = A.heads * A.dim, Nk = A.kv_heads * A.dim, R = L.lru_width, bw = R / L.lru_blocks;
      const int og = Nq + Nk, oy = og + A.heads, ox = oy + R, Nin = ox + R;
      FAM_TRY(KK_F32_PROJ, proj(m->hn, W, L.w_in, W, Nin, m->p0, Nin, n));
      {  // left: normed keys and the raw keys as values go to the cache, the queries are normed in place
        KvStoreArgs ks;
        ks.c = cache_of(A), ks.k = m->p0 + Nq, ks.ldk = Nin, ks.v = m->p0 + Nq, ks.ldv = Nin;
        ks.k_norm = L.k_norm, ks.norm_dim = A.dim, ks.eps = m->eps;
        ks.q = m->p0, ks.ldq = Nin, ks.q_heads = A.heads, ks.q_norm = L.q_norm;
        ks.pos = e->pos_d, ks.slot = e->slot_d, ks.block_table = e->block_table_d, ks.max_pages = e->max_pages_per_seq, ks.n = n;
        FAM_TRY(KK_KV_STORE, launch_kv_store_rows(ks, st));
        GqaAttnArgs g;
        g.q = m->p0, g.ldq = Nin, g.out = m->p1, g.ldo = A.heads * A.vdim;
        g.unit_sink = 1, g.finish = 1, g.gate = m->p0 + og, g.ldg = Nin;
        FAM_TRY(KK_GQA_ATTN, attend(g));
        FAM_TRY(KK_F32_PROJ, proj(m->p1, A.heads * A.vdim, L.wo, A.heads * A.vdim, W, m->y, W, n));
      }
      {  // right: convolution, block-diagonal gates (fp32: they enter the recurrence), scan, projection
        float* state = m->state + L.state_off;
        ConvArgs c;
        c.x = m->p0 + ox, c.ldx = Nin, c.in_bias = L.x_b, c.w = L.conv_w, c.b = L.conv_b, c.channels = R, c.taps = L.lru_taps;
        c.out = m->p2, c.ldo = R, c.tail = state + R, c.slot_stride = m->slot_floats;
        c.seg_start = segs, c.seg_slot = seg_sl, c.n_seg = n_seg, c.n_rows = n;
        FAM_TRY(KK_CONV, launch_causal_conv(c, st));
        if (L.lru_taps > 1) ++e->launches;
        for (int gi = 0; gi < 2; ++gi) {
          GemmF32 g;
          g.A = m->p2, g.lda = R, g.a_batch = bw;
          g.W = gi ? L.ri : L.ra, g.ldw = bw, g.w_batch = (long)bw * bw;
          g.C = m->p3 + (gi ? R : 0), g.ldc = 2 * R, g.c_batch = bw;
          g.bias = gi ? L.ri_b : L.ra_b, g.bias_batch = bw;
          g.M = n, g.N = bw, g.K = bw, g.batches = L.lru_blocks;
          FAM_TRY(KK_LRU_SCAN, launch_gemm_f32(g, st));
        }
        LruArgs s;
        s.zr = m->p3, s.zi = m->p3 + R, s.ldz = 2 * R, s.u = m->p2, s.ldu = R, s.yb = m->p0 + oy, s.ldy = Nin, s.y_bias = L.y_b, s.lam = L.lam_w;
        s.decay_c = 8.0f, s.channels = R, s.out = m->p2, s.ldo = R, s.state = state, s.slot_stride = m->slot_floats;
        s.seg_start = segs, s.seg_slot = seg_sl, s.n_seg = n_seg, s.n_rows = n;
        s.ws = m->scan_ws, s.ws_floats = m->scan_ws_floats;
        FAM_TRY(KK_LRU_SCAN, launch_lru_scan(s, st));
        FAM_TRY(KK_F32_PROJ, proj(m->p2, R, L.wo2, R, W, m->y2, W, n));
      }
      y2 = m->y2, s1 = L.left_scale, s2 = L.right_scale;
    } else {
      const int inner = L.m_heads * L.m_P, GN = L.m_groups * L.m_N, C = inner + 2 * GN, Nin = 2 * inner + 2 * GN + L.m_heads;
      float* state = m->state + L.state_off;
      FAM_TRY(KK_F32_PROJ, proj(m->hn, W, L.w_in, W, Nin, m->p0, Nin, n));
      ConvArgs c;
      c.x = m->p0 + inner, c.ldx = Nin, c.w = L.conv_w, c.b = L.conv_b, c.channels = C, c.taps = L.m_taps, c.act = 1;
      c.out = m->p1, c.ldo = C, c.tail = state + (size_t)L.m_heads * L.m_N * L.m_P, c.slot_stride = m->slot_floats;
      c.seg_start = segs, c.seg_slot = seg_sl, c.n_seg = n_seg, c.n_rows = n;
      FAM_TRY(KK_CONV, launch_causal_conv(c, st));
      if (L.m_taps > 1) ++e->launches;
      SsdArgs s;
      s.x = m->p1, s.B = m->p1 + inner, s.C = m->p1 + inner + GN, s.ld = C, s.dt_raw = m->p0 + 2 * inner + 2 * GN, s.ld_dt = Nin;
      s.dt_bias = L.dt_bias, s.A_log = L.A_log, s.D = L.Dw, s.heads = L.m_heads, s.P = L.m_P, s.N = L.m_N, s.groups = L.m_groups;
      s.y = m->p2, s.ldy = inner, s.state = state, s.slot_stride = m->slot_floats;
      s.seg_start = segs, s.seg_slot = seg_sl, s.n_seg = n_seg, s.n_rows = n;
      s.ws = m->scan_ws, s.ws_floats = m->scan_ws_floats;
      FAM_TRY(KK_SSD_SCAN, launch_ssd_scan(s, st));
      FAM_TRY(KK_F32_NORM, launch_gated_group_norm(m->p2, inner, m->p0, Nin, L.gn_w, m->p3, inner, inner, L.m_norm_groups, m->eps, n, st));
      FAM_TRY(KK_F32_PROJ, proj(m->p3, inner, L.wo, inner, W, m->y, W, n));
    }
    const FvLayer* next = li + 1 < m->layers.size() ? &m->layers[li + 1] : nullptr;
    {  // the mixer's write; the same launch reads for the feed-forward or for the next layer's mixer
      HyperStep hs;
      hs.X = m->X, hs.width = W, hs.streams = S, hs.n = n;
      hs.mix = L.hc1_mix, hs.out = L.hc1_out, hs.y1 = m->y, hs.s1 = s1, hs.y2 = y2, hs.s2 = s2, hs.eps = m->eps;
      if (L.ff > 0) hs.in = L.hc2_in, hs.w = L.norm2, hs.h = m->hn;
      else if (next) hs.in = next->hc1_in, hs.w = next->norm1, hs.h = m->hn;
      FAM_TRY(KK_HYPER, launch_hyper_step(hs, st));
    }
    if (L.ff > 0) {
      FAM_TRY(KK_F32_PROJ, proj(m->hn, W, L.w_gu, W, 2 * L.ff, m->p0, 2 * L.ff, n));
      FAM_TRY(KK_GLU, launch_clamped_glu(m->p0, 2 * L.ff, m->p1, L.ff, L.limit, 1.702f, n, st));
      FAM_TRY(KK_F32_PROJ, proj(m->p1, L.ff, L.w_down, L.ff, W, m->y, W, n));
      HyperStep hs;
      hs.X = m->X, hs.width = W, hs.streams = S, hs.n = n;
      hs.mix = L.hc2_mix, hs.out = L.hc2_out, hs.y1 = m->y, hs.eps = m->eps;
      if (next) hs.in = next->hc1_in, hs.w = next->norm1, hs.h = m->hn;
      FAM_TRY(KK_HYPER, launch_hyper_step(hs, st));
    }
    if (m->dump_layers) {  // parity hook: the sum of the streams after the layer
      HyperStep hs;
      hs.X = m->X, hs.width = W, hs.streams = S, hs.n = n;
      hs.sum_out = m->layer_dump + li * (size_t)e->opts.max_batch_tokens * W;
      FAM_TRY(KK_HYPER, launch_hyper_step(hs, st));
    }
  }
  if (n_out <= 0) return cudaSuccess;
  {
    HyperStep hs;
    hs.X = m->X, hs.width = W, hs.streams = S, hs.n = n_out;
    hs.w = m->final_norm, hs.eps = m->eps, hs.h = m->xo, hs.gather = outs;
    FAM_TRY(KK_F32_NORM, launch_hyper_step(hs, st));
  }
  {
    GemmF32 g;
    g.A = m->xo, g.lda = W, g.W = m->head, g.ldw = W, g.C = m->logits, g.ldc = m->vocab, g.M = n_out, g.N = m->vocab, g.K = W, g.round_a = rnd;
    FAM_TRY(KK_LM_HEAD, launch_gemm_f32(g, st));
  }
  return sample_rows(e, n_out, temperature, advance);
}

}  // namespace qie
