// Host side of hybrid models (xb_hybrid_desc / xb_hybrid_layer in xb200.h): weights by checkpoint name, per-slot
// state (recurrent matrices + filter tails) beside the paged KV pools, and the launch sequence of one forward.
// Included by xb_engine.cu after the definition of xb_engine: batch bookkeeping, page lists, metadata upload,
// CUDA-graph replay of decode steps, sampling and the loader are the engine's own.
#pragma once
#include "xb_hybrid_kernels.cuh"
#include <set>
#include <tuple>

// rows x key shares that the split form of the latent attention may write: steps of fewer than num_sms / 2 tiles of 64 rows
// use it, with at most this many (row, share) pairs
#define HY_LAT_SPLIT_ROWS 4864

struct HyTarget {
  void* dst = nullptr;
  bool f32 = false;          // destination type: fp32 (vectors, filters) or bf16 (matrices, tables)
  long long rows = 0, cols = 0, ld = 0;
  int ndim = 0;
  bool optional = false;     // a tensor the model can run without (nothing reads it); not counted as missing
};

struct HyLayer {
  xb_hybrid_layer d{};
  int n_in = 0;              // rows of the fused input projection
  int off_q = 0, off_k = 0, off_v = 0, off_g = 0, off_b = 0, off_a = 0, off_rq = 0, off_rf = 0, off_rv = 0;
  int c_conv = 0;            // delta: channels that pass the short filter (q | k | v)
  int n_o = 0, n_o2 = 0;     // inputs of the output projection(s)
  bf16 *w_in = nullptr, *w_o = nullptr, *w_o2 = nullptr, *w_up = nullptr, *w_down = nullptr, *w_sgate = nullptr, *w_sproj = nullptr;
  float *b_in = nullptr, *norm1 = nullptr, *norm1b = nullptr, *norm2 = nullptr, *norm2b = nullptr, *canon1 = nullptr,
        *canon2 = nullptr, *side_norm = nullptr, *conv_w = nullptr, *A_log = nullptr, *dt_bias = nullptr, *head_norm = nullptr,
        *lower = nullptr;
  // tile-major copies for the tcgen05 Linear (bf16 serving; made once all weights are in, see hy_finalize)
  bf16 *t_in = nullptr, *t_o = nullptr, *t_o2 = nullptr, *t_up = nullptr, *t_down = nullptr, *t_sgate = nullptr, *t_sproj = nullptr;
  void *k_pool = nullptr, *v_pool = nullptr;
  // bf16 serving, key and value heads of one size (64 or 128) and at most 8 query heads per key head: prompts run through the
  // engine's tcgen05 attention (window and kept first keys as its mask), reading the pools through these tensor maps
  bool tc_attn = false;
  CUtensorMap tmK, tmV;
  size_t st_rec = 0, st_conv = 0, st_canon1 = 0, st_canon2 = 0;   // float offsets inside a slot's state
  // latent attention / general delta rule / lightning and the gated feed-forwards
  int off_dkv = 0, off_r = 0, off_w1 = 0;   // more columns of the fused input projection
  int n_up = 0, n_dn = 0;                   // rows of the fused up projection, inputs of the down projection
  bf16 *w_uk = nullptr, *w_uv = nullptr, *w_d2 = nullptr, *w_router = nullptr, *t_d2 = nullptr;
  float *b_up = nullptr, *b_down = nullptr, *lat_norm = nullptr, *rot_freq = nullptr, *w0 = nullptr, *hdecay = nullptr;
  int owner = -1;                           // layer whose tensors this one uses (weights_of), -1: its own
  // rotary-position attention (XB_MIX_SOFTMAX)
  float *sink = nullptr, *talk = nullptr, *vmix = nullptr;
  double* rot_freq_d = nullptr;             // [s_rot_dims / 2] rescaled frequencies
  int vmode = 0;                            // 0: values as projected; 1: leaves its values for later layers; 2: blends with them
  bool v_all = false;                       // a value row of the pool holds every key head ([page][token][G * dv])
  // whole-projection q / k norm weights, the distance penalty's two numbers per head (XB_MIX_SOFTMAX options)
  float *qn = nullptr, *kn = nullptr, *r1 = nullptr, *r2 = nullptr;
  // gated residual: the gate's rows sit behind the mixer's in w_in (off_rg) and behind the experts' in w_up (off_rg2)
  int off_rg = -1, off_rg2 = -1;
};

struct HyModel {
  xb_hybrid_desc d{};
  std::vector<HyLayer> L;
  bf16 *embed = nullptr, *side_embed = nullptr, *head = nullptr;
  bf16 *bigram = nullptr, *pos_tab = nullptr;   // hashed token-pair rows [buckets + 1, dim], learned position rows [pos_rows, dim]
  size_t st_prev = 0;                           // float offset of a slot's previous token (its bits) inside the slot's state
  float* final_norm = nullptr;
  float* state = nullptr;
  size_t state_floats = 0;   // per slot
  float *x = nullptr, *hn = nullptr, *P = nullptr, *c = nullptr, *o = nullptr, *m1 = nullptr, *m2 = nullptr, *beta = nullptr,
        *decay = nullptr, *qk = nullptr, *head_raw = nullptr;
  void *a1 = nullptr, *a2 = nullptr, *head_in = nullptr;
  bf16* qg = nullptr;        // [T, q | gate] of an attention layer for the tcgen05 kernel (see hy_qg_pack_kernel)
  int* d_ones = nullptr;     // tile lengths of a step of single tokens
  size_t maxQG = 0;
  int* d_rows = nullptr;
  size_t maxN = 0, maxK = 0, maxC = 0, maxO = 0, maxH = 1;
  std::map<std::string, HyTarget> names;
  std::set<std::string> loaded;
  std::vector<void*> allocs;
  bf16* t_head = nullptr;
  bool finalized = false;
  // steps of few rows are chains of short kernels: their launches overlap (programmatic serialization); prompts run long
  // kernels, where blocks of the next kernel parked on the SMs cost more than the launch gap (measured: +17% per prompt)
  float* lat_part = nullptr;           // latent attention: (max, sum, accumulator) of every key share [splits][rows][2 + rank]
  int use_lat_mma = 1;                 // XB_HY_LAT_MMA: 0 = latent attention through the per-(token, head) kernel everywhere (A/B)
  size_t maxLatR = 0;
  float *qa = nullptr, *gw = nullptr;   // latent attention: queries in the cache's space [T, H * (rank + rot)]; experts: weights [T, E]
  void* ah = nullptr;                  // parallel blocks: the normed stream as a Linear input (both sublayers read it)
  size_t maxQA = 0, maxE = 0, maxM = 0;   // maxM: widest matrix that passes through the m1 / m2 buffers besides the stream's width
  float* vfirst = nullptr;              // values of the first blending layer for the tokens of this step [T, G * dv]
  size_t maxGV = 0;
  int use_gather = 1;                   // XB_HY_GATHER=0: experts always as one wide Linear pair (A/B)
  int fuse_router = 1;                  // XB_HY_FUSE_ROUTER=0: steps of few rows form the router's logits and route in two kernels (A/B)
  int p_split = 1;                      // XB_HY_P_SPLIT=0: rotary-position attention rounds its softmax weights to bf16 (A/B)
  int dec_splits = 1;                   // key splits of this step's single-token attention (hy_kv_splits)
  bool pdl_now = false;
  int recur_lpc = 0;         // XB_HY_LPC=4|8|16 pins the lanes per state column (A/B); 0: by the step's shape
  int use_tc_attn = 1;       // XB_HY_TC_ATTN=0: attention through the per-token kernel everywhere (A/B)
  int use_tc = 1;            // XB_HY_TC=0: every Linear through the plain kernels (A/B)
  size_t cap_P = 0, cap_m = 0, cap_head = 0;   // bytes of the Linear output buffers
  std::map<std::tuple<const void*, const void*, const void*, int>, GemmPlan> plans;
};

static int* hy_rows_buffer(xb_engine* e) { return e->hy->d_rows; }
static int hy_max_rows(xb_engine* e) { return e->hy->d.max_logit_rows > e->hy->d.max_seqs ? e->hy->d.max_logit_rows : e->hy->d.max_seqs; }

static void hy_drop_plans(xb_engine* e) { e->hy->plans.clear(); }

static int hy_alloc(HyModel* hy, void** p, size_t bytes) {
  XB_TRY(dmalloc(p, bytes));
  XB_CUDA(cudaMemset(*p, 0, bytes ? bytes : 16));
  hy->allocs.push_back(*p);
  return 0;
}
template <typename T>
static int hy_alloc_t(HyModel* hy, T** p, size_t n) { return hy_alloc(hy, (void**)p, n * sizeof(T)); }

static void hy_name(HyModel* hy, const std::string& name, void* dst, bool f32, long long rows, long long cols, long long ld, int ndim) {
  HyTarget t;
  t.dst = dst; t.f32 = f32; t.rows = rows; t.cols = cols; t.ld = ld; t.ndim = ndim;
  hy->names[name] = t;
}
// a matrix that occupies rows [row0, row0 + rows) of a fused bf16 matrix with K columns
static void hy_name_rows(HyModel* hy, const std::string& name, bf16* base, long long row0, long long rows, long long K) {
  hy_name(hy, name, base + row0 * K, false, rows, K, K, 2);
}
static void hy_name_vec(HyModel* hy, const std::string& name, float* dst, long long n) { hy_name(hy, name, dst, true, 1, n, n, 1); }

static void hy_destroy(HyModel* hy) {
  if (hy == nullptr) return;
  for (void* p : hy->allocs) cudaFree(p);
  for (HyLayer& l : hy->L) {
    cudaFree(l.k_pool); cudaFree(l.v_pool);
    if (l.owner >= 0) continue;   // the tile-major copies belong to the layer that owns the tensors
    cudaFree(l.t_in); cudaFree(l.t_o); cudaFree(l.t_o2); cudaFree(l.t_up); cudaFree(l.t_down); cudaFree(l.t_sgate); cudaFree(l.t_sproj);
    cudaFree(l.t_d2);
  }
  cudaFree(hy->t_head);
  cudaFree(hy->state);
  delete hy;
}

// A matrix that occupies columns [col0, col0 + cols) of a fused bf16 matrix with `ld` columns (the down projections of
// experts side by side are ONE matrix over all experts' activations).
static void hy_name_cols(HyModel* hy, const std::string& name, bf16* base, long long col0, long long rows, long long cols, long long ld) {
  hy_name(hy, name, base + col0, false, rows, cols, ld, 2);
}

// Mixers of the parallel-block designs.  own: the layer has tensors of its own (else only cache / state is laid out).
static int hy_create_mixer(xb_engine* e, int i, bool own, size_t& st, uint64_t& wbytes, uint64_t& kvpos) {
  HyModel* hy = e->hy;
  HyLayer& l = hy->L[i];
  const xb_hybrid_layer& c = l.d;
  const xb_hybrid_desc& d = hy->d;
  const size_t D = d.dim;
  const std::string p = "l" + std::to_string(i) + ".mix.";
  const long long H = c.m_heads, n = c.m_dim;
  XB_CHECK(H > 0 && n > 0, "layer %d: bad mixer sizes", i);
  if (c.mixer == XB_MIX_LATENT) {
    const long long dr = c.m_rot_dim, dv = c.m_vdim, R = c.m_kv_rank;
    XB_CHECK(dr >= 0 && dv > 0 && R > 0 && R <= 512, "layer %d: bad latent attention sizes (latent of at most 512 numbers)", i);
    XB_CHECK(c.m_rot_dims >= 0 && c.m_rot_dims <= dr && c.m_rot_dims % 2 == 0, "layer %d: %d rotating entries do not fit a part of %lld", i,
             c.m_rot_dims, dr);
    l.off_q = 0; l.off_dkv = (int)(H * (n + dr));
    l.n_in = l.off_dkv + (int)(R + dr);
    if (d.gated_residual) { l.off_rg = l.n_in; l.n_in += (int)D; }
    l.n_o = (int)(H * dv);
    if (own) {
      XB_TRY(hy_alloc_t(hy, &l.w_in, (size_t)l.n_in * D));
      if (d.gated_residual) XB_TRY(hy_alloc_t(hy, &l.b_in, (size_t)l.n_in));
      XB_TRY(hy_alloc_t(hy, &l.w_o, D * l.n_o));
      XB_TRY(hy_alloc_t(hy, &l.w_uk, (size_t)(H * n * R)));
      XB_TRY(hy_alloc_t(hy, &l.w_uv, (size_t)(H * dv * R)));
      XB_TRY(hy_alloc_t(hy, &l.lat_norm, (size_t)R));
      hy_name_rows(hy, p + "q", l.w_in, l.off_q, H * (n + dr), D);
      hy_name_rows(hy, p + "dkv", l.w_in, l.off_dkv, R + dr, D);
      hy_name_vec(hy, p + "dkv.norm", l.lat_norm, R);
      hy_name_rows(hy, p + "uk", l.w_uk, 0, H * n, R);
      hy_name_rows(hy, p + "uv", l.w_uv, 0, H * dv, R);
      hy_name_rows(hy, p + "o", l.w_o, 0, D, l.n_o);
      const int half = c.m_rot_dims / 2;
      std::vector<float> fr((size_t)(half > 0 ? half : 1), 0.f);
      for (int j = 0; j < half; ++j) fr[j] = (float)pow((double)c.m_rot_base, -2.0 * j / (double)c.m_rot_dims);
      XB_TRY(hy_alloc_t(hy, &l.rot_freq, fr.size()));
      XB_CUDA(cudaMemcpy(l.rot_freq, fr.data(), fr.size() * sizeof(float), cudaMemcpyHostToDevice));
      wbytes += ((size_t)l.n_in * D + D * l.n_o + (size_t)(H * (n + dv) * R)) * 2;
    }
    const size_t qa = (size_t)(H * (R + dr)), ol = (size_t)(H * R);
    if (qa > hy->maxQA) hy->maxQA = qa;
    if ((size_t)R > hy->maxLatR) hy->maxLatR = R;
    if (ol > hy->maxO) hy->maxO = ol;
    kvpos += (uint64_t)(R + dr) * (d.compute_fp32 ? 4 : 2);
  } else if (c.mixer == XB_MIX_GDELTA) {
    const long long HN = H * n, rk = c.m_rank;
    XB_CHECK(n <= HY_MAX_KDIM && rk > 0, "layer %d: bad delta-rule sizes (key dim <= %d)", i, HY_MAX_KDIM);
    l.off_r = 0; l.off_k = (int)HN; l.off_v = (int)(2 * HN); l.off_g = (int)(3 * HN); l.off_a = (int)(4 * HN); l.off_w1 = (int)(5 * HN);
    l.n_in = l.off_w1 + (int)rk;
    l.n_o = (int)HN;
    if (own) {
      XB_TRY(hy_alloc_t(hy, &l.w_in, (size_t)l.n_in * D));
      XB_TRY(hy_alloc_t(hy, &l.b_in, (size_t)l.n_in));
      XB_TRY(hy_alloc_t(hy, &l.w_o, D * l.n_o));
      XB_TRY(hy_alloc_t(hy, &l.w_d2, (size_t)(HN * rk)));
      XB_TRY(hy_alloc_t(hy, &l.w0, (size_t)HN));
      XB_TRY(hy_alloc_t(hy, &l.head_norm, (size_t)HN));
      hy_name_rows(hy, p + "r", l.w_in, l.off_r, HN, D);
      hy_name_rows(hy, p + "k", l.w_in, l.off_k, HN, D);
      hy_name_rows(hy, p + "v", l.w_in, l.off_v, HN, D);
      hy_name_rows(hy, p + "g", l.w_in, l.off_g, HN, D);
      hy_name_rows(hy, p + "a", l.w_in, l.off_a, HN, D);   hy_name_vec(hy, p + "a.b", l.b_in + l.off_a, HN);
      hy_name_rows(hy, p + "w1", l.w_in, l.off_w1, rk, D);
      hy_name_rows(hy, p + "w2", l.w_d2, 0, HN, rk);
      hy_name_vec(hy, p + "w0", l.w0, HN);
      hy_name_vec(hy, p + "norm", l.head_norm, HN);
      hy_name_rows(hy, p + "o", l.w_o, 0, D, l.n_o);
      wbytes += ((size_t)l.n_in * D + D * l.n_o + (size_t)(HN * rk)) * 2;
    }
    l.st_rec = st; st += (size_t)(HN * n);
    if ((size_t)H > hy->maxH) hy->maxH = H;
    if ((size_t)(6 * HN) > hy->maxC) hy->maxC = 6 * HN;
    if ((size_t)l.n_o > hy->maxO) hy->maxO = l.n_o;
    if ((size_t)rk > hy->maxK) hy->maxK = rk;
    if ((size_t)HN > hy->maxM) hy->maxM = HN;
  } else {
    const long long dv = c.m_vdim;
    XB_CHECK(n <= HY_MAX_KDIM && dv > 0, "layer %d: bad lightning sizes (key dim <= %d)", i, HY_MAX_KDIM);
    l.off_q = 0; l.off_k = (int)(H * n); l.off_v = (int)(2 * H * n); l.off_g = l.off_v + (int)(H * dv);
    l.n_in = l.off_g + (int)(H * dv);
    l.n_o = (int)(H * dv);
    if (own) {
      XB_TRY(hy_alloc_t(hy, &l.w_in, (size_t)l.n_in * D));
      XB_TRY(hy_alloc_t(hy, &l.w_o, D * l.n_o));
      XB_TRY(hy_alloc_t(hy, &l.head_norm, (size_t)(H * dv)));
      XB_TRY(hy_alloc_t(hy, &l.hdecay, (size_t)H));
      hy_name_rows(hy, p + "q", l.w_in, l.off_q, H * n, D);
      hy_name_rows(hy, p + "k", l.w_in, l.off_k, H * n, D);
      hy_name_rows(hy, p + "v", l.w_in, l.off_v, H * dv, D);
      hy_name_rows(hy, p + "g", l.w_in, l.off_g, H * dv, D);
      hy_name_vec(hy, p + "norm", l.head_norm, H * dv);
      hy_name_vec(hy, p + "decay", l.hdecay, H);       // from the configuration, not the checkpoint
      hy_name_rows(hy, p + "o", l.w_o, 0, D, l.n_o);
      wbytes += ((size_t)l.n_in * D + D * l.n_o) * 2;
    }
    l.st_rec = st; st += (size_t)(H * dv * n);
    const size_t cc = (size_t)(2 * H * n + H * dv);
    if (cc > hy->maxC) hy->maxC = cc;
    if ((size_t)l.n_o > hy->maxO) hy->maxO = l.n_o;
  }
  return 0;
}

// Rotary-position softmax attention: q | k | v | head gates are the rows of one input matrix; sink, head-mixing matrix and
// blend factor are fp32 vectors; the rescaled rotary frequencies are made here, in double, from the layer's constants.
static int hy_create_softmax(xb_engine* e, int i, bool own, uint64_t& wbytes, uint64_t& kvpos) {
  HyModel* hy = e->hy;
  HyLayer& l = hy->L[i];
  const xb_hybrid_layer& c = l.d;
  const xb_hybrid_desc& d = hy->d;
  const size_t D = d.dim;
  const std::string p = "l" + std::to_string(i) + ".mix.";
  const long long H = c.s_heads, G = c.s_kv_heads, dk = c.s_dim, dv = c.s_vdim, rd = c.s_rot_dims;
  XB_CHECK(own, "layer %d: an attention layer keeps tensors of its own", i);
  XB_CHECK(d.block == XB_BLOCK_SANDWICH || d.block == XB_BLOCK_BRANCHNORM, "layer %d: softmax attention belongs to sandwich or branch-norm blocks", i);
  XB_CHECK(H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0, "layer %d: bad attention sizes", i);
  const bool vk = c.s_v_is_k != 0;
  const bool prep2 = c.s_qk_norm != 0 || vk || c.s_qtemp_every > 0;   // hy_qk_prep_kernel in place of the rotation kernel
  XB_CHECK(!vk || (dv == dk && !c.s_vmix && !c.s_talk), "layer %d: values that are the keys need equal sizes and neither blending nor mixed heads", i);
  XB_CHECK(!prep2 || (rd == 0 && !c.s_vmix && !c.s_talk), "layer %d: whole-projection norms, key values and the query temperature come without rotation, blending or mixed heads", i);
  XB_CHECK(!prep2 || (size_t)((H + G) * dk) * sizeof(float) <= 48 * 1024, "layer %d: %lld query and key channels per token (at most 12288)", i, (H + G) * dk);
  XB_CHECK(c.s_qtemp_every >= 0 && c.s_sink >= XB_SINK_NONE && c.s_sink <= XB_SINK_UNIT, "layer %d: bad query temperature step %d / sink kind %d", i, c.s_qtemp_every, c.s_sink);
  XB_CHECK(rd >= 0 && rd <= dk && rd % 2 == 0, "layer %d: %lld rotating entries do not fit a head of %lld", i, rd, dk);
  XB_CHECK(rd / 2 <= HY_MAX_ROT_PAIRS, "layer %d: %lld rotating entries (at most %d)", i, rd, 2 * HY_MAX_ROT_PAIRS);
  XB_CHECK(c.s_rot_pairs == XB_ROPE_INTERLEAVED || c.s_rot_pairs == XB_ROPE_HALF_SPLIT, "layer %d: unknown rotary pair layout %d", i, c.s_rot_pairs);
  XB_CHECK(c.s_softcap >= 0.f && c.s_scale > 0.f, "layer %d: bad score scale %g / soft cap %g", i, c.s_scale, c.s_softcap);
  l.v_all = c.s_talk != 0 && G > 1;
  const long long dvo = l.v_all ? G * dv : dv;   // value channels one (token, head) block of the attention kernel carries
  // values that are the keys as projected: no value rows, the value columns ARE the key columns
  l.off_q = 0; l.off_k = (int)(H * dk); l.off_v = vk ? l.off_k : l.off_k + (int)(G * dk); l.off_g = l.off_v + (int)(G * dv);
  l.n_in = l.off_g + (c.s_gate ? (int)H : 0);
  if (d.gated_residual) { l.off_rg = l.n_in; l.n_in += (int)D; }
  l.n_o = (int)(H * dv);
  XB_TRY(hy_alloc_t(hy, &l.w_in, (size_t)l.n_in * D));
  XB_TRY(hy_alloc_t(hy, &l.w_o, D * l.n_o));
  hy_name_rows(hy, p + "q", l.w_in, l.off_q, H * dk, D);
  hy_name_rows(hy, p + "k", l.w_in, l.off_k, G * dk, D);
  if (!vk) hy_name_rows(hy, p + "v", l.w_in, l.off_v, G * dv, D);
  if (c.s_gate) hy_name_rows(hy, p + "g", l.w_in, l.off_g, H, D);
  hy_name_rows(hy, p + "o", l.w_o, 0, D, l.n_o);
  if (c.s_qkv_bias || d.gated_residual) XB_TRY(hy_alloc_t(hy, &l.b_in, (size_t)l.n_in));
  if (c.s_qkv_bias) {
    hy_name_vec(hy, p + "q.b", l.b_in + l.off_q, H * dk);
    hy_name_vec(hy, p + "k.b", l.b_in + l.off_k, G * dk);
    if (!vk) hy_name_vec(hy, p + "v.b", l.b_in + l.off_v, G * dv);
  }
  if (c.s_qk_norm) {
    XB_TRY(hy_alloc_t(hy, &l.qn, (size_t)(H * dk))); hy_name_vec(hy, p + "q.norm", l.qn, H * dk);
    XB_TRY(hy_alloc_t(hy, &l.kn, (size_t)(G * dk))); hy_name_vec(hy, p + "k.norm", l.kn, G * dk);
  }
  if (c.s_dist_bias) {
    XB_TRY(hy_alloc_t(hy, &l.r1, (size_t)H)); hy_name_vec(hy, p + "r1", l.r1, H);
    XB_TRY(hy_alloc_t(hy, &l.r2, (size_t)H)); hy_name_vec(hy, p + "r2", l.r2, H);
  }
  if (c.s_sink == XB_SINK_LEARNED) { XB_TRY(hy_alloc_t(hy, &l.sink, (size_t)H)); hy_name_vec(hy, p + "sink", l.sink, H); }
  if (c.s_sink == XB_SINK_UNIT) XB_TRY(hy_alloc_t(hy, &l.sink, (size_t)H));   // a sink of score 0 per head: the zeros the allocation leaves
  if (c.s_talk) { XB_TRY(hy_alloc_t(hy, &l.talk, (size_t)(H * H))); hy_name(hy, p + "talk", l.talk, true, H, H, H, 2); }
  if (c.s_vmix) { XB_TRY(hy_alloc_t(hy, &l.vmix, 1)); hy_name_vec(hy, p + "vmix", l.vmix, 1); }
  // frequencies f_j = base^(-2j/dims), rescaled (xb200.h: XB_ROT_SCALE_*)
  const int half = (int)(rd / 2);
  std::vector<double> fr((size_t)(half > 0 ? half : 1), 0.0);
  const double base = c.s_rot_base, fac = c.s_rot_factor, orig = c.s_rot_orig, p0 = c.s_rot_p0, p1 = c.s_rot_p1;
  const double two_pi = 6.283185307179586476925286766559;
  XB_CHECK(half == 0 || base > 1.0, "layer %d: rotary base %g", i, base);
  XB_CHECK(c.s_rot_scaling == XB_ROT_SCALE_NONE || (fac > 0.0 && orig > 0.0), "layer %d: bad rotary scaling constants", i);
  double lo = 0.0, hi = 0.0;
  if (c.s_rot_scaling == XB_ROT_SCALE_RAMP && half > 0) {
    XB_CHECK(p0 > 0.0 && p1 > 0.0, "layer %d: bad rotary ramp constants", i);
    auto at = [&](double t) { return (double)rd * log(orig / (two_pi * t)) / (2.0 * log(base)); };
    lo = floor(at(p0)); lo = lo < 0.0 ? 0.0 : lo;
    hi = ceil(at(p1)); hi = hi > (double)(rd - 1) ? (double)(rd - 1) : hi;
  }
  for (int j = 0; j < half; ++j) {
    double f = pow(base, -2.0 * j / (double)rd);
    if (c.s_rot_scaling == XB_ROT_SCALE_BANDS) {
      XB_CHECK(p1 != p0 && p0 > 0.0 && p1 > 0.0, "layer %d: bad rotary band constants", i);
      const double wl = two_pi / f;
      if (wl < orig / p1) { /* kept */ }
      else if (wl > orig / p0) f = f / fac;
      else { const double sm = (orig / wl - p0) / (p1 - p0); f = (1.0 - sm) * f / fac + sm * f; }
    } else if (c.s_rot_scaling == XB_ROT_SCALE_RAMP) {
      double r = ((double)j - lo) / (hi - lo > 0.001 ? hi - lo : 0.001);
      r = r < 0.0 ? 0.0 : (r > 1.0 ? 1.0 : r);
      f = f / fac * r + f * (1.0 - r);
    } else {
      XB_CHECK(c.s_rot_scaling == XB_ROT_SCALE_NONE, "layer %d: unknown rotary scaling %d", i, c.s_rot_scaling);
    }
    fr[j] = f;
  }
  XB_TRY(hy_alloc_t(hy, &l.rot_freq_d, fr.size()));
  XB_CUDA(cudaMemcpy(l.rot_freq_d, fr.data(), fr.size() * sizeof(double), cudaMemcpyHostToDevice));
  const size_t qa = (size_t)(H * dk), ol = (size_t)(H * dvo);
  if (qa > hy->maxQA) hy->maxQA = qa;
  if (ol > hy->maxO) hy->maxO = ol;
  if (c.s_vmix && (size_t)(G * dv) > hy->maxGV) hy->maxGV = (size_t)(G * dv);
  // bf16 serving, key and value heads of one size (64 or 128), at most 8 query heads per key head: prompts run through the
  // engine's tcgen05 attention (sink, score cap and the wide value rows of mixed heads as its options)
  l.tc_attn = !d.compute_fp32 && dk == dv && (dk == 64 || dk == 128) && H / G <= 8;
  if (l.tc_attn && qa > hy->maxQG) hy->maxQG = qa;
  wbytes += ((size_t)l.n_in * D + D * l.n_o) * 2;
  kvpos += (uint64_t)G * (dk + dv) * (d.compute_fp32 ? 4 : 2);
  return 0;
}

// Gated feed-forwards: dense (gate | up rows of one matrix, biases) or experts (every expert's gate | up rows, then the
// shared expert's, in one matrix; every expert's down projection side by side as the columns of one matrix).
static int hy_create_ff(xb_engine* e, int i, bool own, uint64_t& wbytes) {
  HyModel* hy = e->hy;
  HyLayer& l = hy->L[i];
  const xb_hybrid_layer& c = l.d;
  const size_t D = hy->d.dim, F = c.ff;
  const std::string p = "l" + std::to_string(i) + ".mlp.";
  XB_CHECK(hy->d.block == XB_BLOCK_PARALLEL || c.ff_kind == XB_FF_MOE, "layer %d: the dense gated feed-forward belongs to parallel blocks", i);
  XB_CHECK(c.ff_act == XB_ACT_GLU_CLAMP || c.ff_act == XB_ACT_SWIGLU || c.ff_act == XB_ACT_GELU, "layer %d: unknown expert activation %d", i, c.ff_act);
  XB_CHECK(c.ff_act != XB_ACT_GELU || (c.ff_kind == XB_FF_MOE && !c.route_input), "layer %d: the ungated GELU form serves experts weighted on their output", i);
  XB_CHECK((c.route_score == XB_ROUTE_SIGMOID || c.route_score == XB_ROUTE_SOFTMAX) && (c.group_score == XB_GROUP_TOP2 || c.group_score == XB_GROUP_MAX),
           "layer %d: unknown router score %d / group score %d", i, c.route_score, c.group_score);
  const bool rg = hy->d.gated_residual != 0;
  if (c.ff_kind == XB_FF_GLU_CLAMP) {
    l.n_up = (int)(2 * F); l.n_dn = (int)F;
    if (own) {
      XB_TRY(hy_alloc_t(hy, &l.w_up, (size_t)l.n_up * D));
      XB_TRY(hy_alloc_t(hy, &l.b_up, (size_t)l.n_up));
      XB_TRY(hy_alloc_t(hy, &l.w_down, D * F));
      XB_TRY(hy_alloc_t(hy, &l.b_down, D));
      hy_name_rows(hy, p + "gate", l.w_up, 0, F, D);   hy_name_vec(hy, p + "gate.b", l.b_up, F);
      hy_name_rows(hy, p + "up", l.w_up, F, F, D);     hy_name_vec(hy, p + "up.b", l.b_up + F, F);
      hy_name_rows(hy, p + "down", l.w_down, 0, D, F); hy_name_vec(hy, p + "down.b", l.b_down, D);
    }
  } else if (c.ff_kind == XB_FF_MOE) {
    const size_t E = c.n_experts, S = c.shared_ff > 0 ? c.shared_ff : 0;
    XB_CHECK(E > 0 && c.top > 0 && (size_t)c.top <= E, "layer %d: %d experts, %d per token", i, c.n_experts, c.top);
    XB_CHECK(c.groups == 0 || (c.groups > 0 && E % c.groups == 0 && c.keep_groups > 0 && c.keep_groups <= c.groups &&
                               (size_t)c.top <= (E / c.groups) * c.keep_groups),
             "layer %d: %d groups (%d kept) do not fit %d experts with %d per token", i, c.groups, c.keep_groups, c.n_experts, c.top);
    const bool gated = c.ff_act != XB_ACT_GELU;   // ungated experts: up rows only, expert after expert, then the shared expert's
    const size_t U = gated ? 2 : 1;
    l.n_up = (int)(U * (E * F + S)); l.n_dn = (int)(E * F + S);
    if (rg) { l.off_rg2 = l.n_up; l.n_up += (int)D; }   // the residual gate reads what the experts read: its rows follow theirs
    if (own) {
      XB_TRY(hy_alloc_t(hy, &l.w_up, (size_t)l.n_up * D));
      XB_TRY(hy_alloc_t(hy, &l.w_down, D * l.n_dn));
      XB_TRY(hy_alloc_t(hy, &l.w_router, E * D));
      hy_name_rows(hy, p + "router", l.w_router, 0, E, D);
      for (size_t x = 0; x < E; ++x) {
        const std::string pe = p + "e" + std::to_string(x) + ".";
        if (gated) hy_name_rows(hy, pe + "gate", l.w_up, 2 * x * F, F, D);
        hy_name_rows(hy, pe + "up", l.w_up, gated ? 2 * x * F + F : x * F, F, D);
        hy_name_cols(hy, pe + "down", l.w_down, x * F, D, F, l.n_dn);
      }
      if (S > 0) {
        if (gated) hy_name_rows(hy, p + "shared.gate", l.w_up, 2 * E * F, S, D);
        hy_name_rows(hy, p + "shared.up", l.w_up, gated ? 2 * E * F + S : E * F, S, D);
        hy_name_cols(hy, p + "shared.down", l.w_down, E * F, D, S, l.n_dn);
      }
      if (rg) {
        const std::string pl = "l" + std::to_string(i) + ".";
        XB_TRY(hy_alloc_t(hy, &l.b_up, (size_t)l.n_up));
        hy_name_rows(hy, pl + "rg2", l.w_up, l.off_rg2, D, D);
        hy_name_vec(hy, pl + "rg2.b", l.b_up + l.off_rg2, D);
      }
      wbytes += E * D * 2;
    }
    if (E > hy->maxE) hy->maxE = E;
    if (E > hy->maxM) hy->maxM = E;
  } else {
    return xb_fail(1, "layer %d: unknown feed-forward kind %d", i, c.ff_kind);
  }
  if (own) wbytes += ((size_t)l.n_up * D + D * l.n_dn) * 2;
  if ((size_t)l.n_up > hy->maxN) hy->maxN = l.n_up;
  if ((size_t)l.n_dn > hy->maxK) hy->maxK = l.n_dn;
  return 0;
}

static int hy_create(xb_engine* e, const xb_hybrid_desc& d, const xb_hybrid_layer* layers) {
  HyModel* hy = new HyModel();
  e->hy = hy;
  hy->d = d;
  hy->L.resize(d.n_layers);
  const size_t D = d.dim, Tm = d.max_batch_tokens;
  const int ct = d.taps;
  size_t st = 0;
  uint64_t wbytes = 0, kvpos = 0;
  hy->maxN = D; hy->maxK = D; hy->maxC = 1; hy->maxO = 1;
  if (d.side_dim > 0) { if ((size_t)d.side_dim > hy->maxN) hy->maxN = d.side_dim; if ((size_t)d.side_dim > hy->maxK) hy->maxK = d.side_dim; }
  for (int i = 0; i < d.n_layers; ++i) {
    HyLayer& l = hy->L[i];
    l.d = layers[i];
    const xb_hybrid_layer& c = l.d;
    const std::string p = "l" + std::to_string(i) + ".";
    const bool own = c.weights_of < 0;
    const bool sandwich = d.block == XB_BLOCK_SANDWICH, branchnorm = d.block == XB_BLOCK_BRANCHNORM;
    l.owner = -1;
    XB_CHECK(!branchnorm || (own && (c.mixer == XB_MIX_SOFTMAX || c.mixer == XB_MIX_LATENT) && (c.ff == 0 || c.ff_kind == XB_FF_MOE)),
             "layer %d: branch-norm blocks take softmax or latent attention and experts, with tensors of their own", i);
    if (!own) {
      XB_CHECK(c.weights_of < d.n_layers && c.weights_of != i && layers[c.weights_of].weights_of < 0,
               "layer %d: weights_of %d must name another layer that owns its tensors", i, c.weights_of);
      const xb_hybrid_layer& o = layers[c.weights_of];
      XB_CHECK(o.mixer == c.mixer && o.ff == c.ff && o.ff_kind == c.ff_kind, "layer %d: its description differs from layer %d's, whose tensors it uses",
               i, c.weights_of);
      l.owner = c.weights_of;
    }
    XB_CHECK(own || (c.mixer != XB_MIX_DELTA && c.mixer != XB_MIX_PARALLEL && c.mixer != XB_MIX_SOFTMAX), "layer %d: this mixer kind keeps tensors of its own", i);
    const size_t nd = d.norm_scalar ? 1 : D;   // numbers in a norm of the stream
    if (own) {
      XB_TRY(hy_alloc_t(hy, &l.norm1, nd));
      hy_name_vec(hy, p + "norm1", l.norm1, nd);
      if (sandwich) { XB_TRY(hy_alloc_t(hy, &l.norm1b, D)); hy_name_vec(hy, p + "norm1b", l.norm1b, D); }
    }
    if (ct > 0) {
      if (own) { XB_TRY(hy_alloc_t(hy, &l.canon1, D * ct)); hy_name(hy, p + "canon1", l.canon1, true, D, ct, ct, 2); }
      l.st_canon1 = st; st += (size_t)(ct - 1) * D;
    }
    if (c.mixer == XB_MIX_DELTA) {
      const long long H = c.d_heads, G = c.d_kv_heads, dk = c.d_dim, dv = c.d_vdim, tp = c.d_taps;
      XB_CHECK(H > 0 && G > 0 && H % G == 0 && dk > 0 && dk <= HY_MAX_KDIM && dv > 0, "layer %d: bad delta-rule sizes (key dim <= %d)", i, HY_MAX_KDIM);
      XB_CHECK(tp >= 1 && tp <= HY_MAX_TAPS, "layer %d: short filter of %lld taps (1..%d)", i, tp, HY_MAX_TAPS);
      l.off_q = 0; l.off_k = (int)(G * dk); l.off_v = (int)(2 * G * dk);
      l.c_conv = (int)(2 * G * dk + H * dv);
      l.off_g = l.c_conv; l.off_b = l.off_g + (int)(H * dv); l.off_a = l.off_b + (int)H;
      l.n_in = l.off_a + (int)H;
      l.n_o = (int)(H * dv);
      XB_TRY(hy_alloc_t(hy, &l.w_in, (size_t)l.n_in * D));
      XB_TRY(hy_alloc_t(hy, &l.b_in, (size_t)l.n_in));
      XB_TRY(hy_alloc_t(hy, &l.w_o, D * l.n_o));
      XB_TRY(hy_alloc_t(hy, &l.conv_w, (size_t)l.c_conv * tp));
      XB_TRY(hy_alloc_t(hy, &l.A_log, (size_t)H));
      XB_TRY(hy_alloc_t(hy, &l.dt_bias, (size_t)H));
      XB_TRY(hy_alloc_t(hy, &l.head_norm, (size_t)dv));
      hy_name_rows(hy, p + "mix.q", l.w_in, l.off_q, G * dk, D);
      hy_name_rows(hy, p + "mix.k", l.w_in, l.off_k, G * dk, D);
      hy_name_rows(hy, p + "mix.v", l.w_in, l.off_v, H * dv, D);
      hy_name_rows(hy, p + "mix.g", l.w_in, l.off_g, H * dv, D);
      hy_name_rows(hy, p + "mix.b", l.w_in, l.off_b, H, D);
      hy_name_rows(hy, p + "mix.a", l.w_in, l.off_a, H, D);
      hy_name(hy, p + "mix.q.conv", l.conv_w + (size_t)l.off_q * tp, true, G * dk, tp, tp, 2);
      hy_name(hy, p + "mix.k.conv", l.conv_w + (size_t)l.off_k * tp, true, G * dk, tp, tp, 2);
      hy_name(hy, p + "mix.v.conv", l.conv_w + (size_t)l.off_v * tp, true, H * dv, tp, tp, 2);
      hy_name_vec(hy, p + "mix.A_log", l.A_log, H);
      hy_name_vec(hy, p + "mix.dt_bias", l.dt_bias, H);
      hy_name_vec(hy, p + "mix.norm", l.head_norm, dv);
      hy_name_rows(hy, p + "mix.o", l.w_o, 0, D, l.n_o);
      l.st_rec = st; st += (size_t)(H * dv * dk);
      if ((size_t)H > hy->maxH) hy->maxH = H;
      l.st_conv = st; st += (size_t)(tp - 1) * l.c_conv;
      if ((size_t)l.c_conv > hy->maxC) hy->maxC = l.c_conv;
      if ((size_t)l.n_o > hy->maxO) hy->maxO = l.n_o;
      wbytes += ((size_t)l.n_in * D + D * l.n_o) * 2;
    } else if (c.mixer == XB_MIX_PARALLEL) {
      const long long H = c.a_heads, G = c.a_kv_heads, dk = c.a_dim, dv = c.a_vdim;
      const long long Hr = c.r_heads, rk = c.r_dim, rv = c.r_vdim;
      XB_CHECK(H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0 && dv <= 256, "layer %d: bad attention sizes (value dim <= 256)", i);
      XB_CHECK(c.a_window >= 1 && c.a_keep_first >= 0, "layer %d: bad window %d / kept first tokens %d", i, c.a_window, c.a_keep_first);
      XB_CHECK(Hr > 0 && rk > 0 && rk <= HY_MAX_KDIM && rv > 0, "layer %d: bad HGRN2 sizes (key dim <= %d)", i, HY_MAX_KDIM);
      l.off_q = 0; l.off_k = (int)(H * dk); l.off_v = l.off_k + (int)(G * dk); l.off_g = l.off_v + (int)(G * dv);
      l.off_rq = l.off_g + (int)(H * dv); l.off_rf = l.off_rq + (int)(Hr * rk); l.off_rv = l.off_rf + (int)(Hr * rk);
      l.n_in = l.off_rv + (int)(Hr * rv);
      l.n_o = (int)(H * dv); l.n_o2 = (int)(Hr * rv);
      XB_TRY(hy_alloc_t(hy, &l.w_in, (size_t)l.n_in * D));
      XB_TRY(hy_alloc_t(hy, &l.b_in, (size_t)l.n_in));
      XB_TRY(hy_alloc_t(hy, &l.w_o, D * l.n_o));
      XB_TRY(hy_alloc_t(hy, &l.w_o2, D * l.n_o2));
      XB_TRY(hy_alloc_t(hy, &l.lower, (size_t)(Hr * rk)));
      XB_TRY(hy_alloc_t(hy, &l.head_norm, (size_t)rv));
      hy_name_rows(hy, p + "mix.left.q", l.w_in, l.off_q, H * dk, D);   hy_name_vec(hy, p + "mix.left.q.b", l.b_in + l.off_q, H * dk);
      hy_name_rows(hy, p + "mix.left.k", l.w_in, l.off_k, G * dk, D);   hy_name_vec(hy, p + "mix.left.k.b", l.b_in + l.off_k, G * dk);
      hy_name_rows(hy, p + "mix.left.v", l.w_in, l.off_v, G * dv, D);   hy_name_vec(hy, p + "mix.left.v.b", l.b_in + l.off_v, G * dv);
      hy_name_rows(hy, p + "mix.left.g", l.w_in, l.off_g, H * dv, D);
      hy_name_rows(hy, p + "mix.left.o", l.w_o, 0, D, l.n_o);
      hy_name_rows(hy, p + "mix.right.q", l.w_in, l.off_rq, Hr * rk, D);
      hy_name_rows(hy, p + "mix.right.f", l.w_in, l.off_rf, Hr * rk, D); hy_name_vec(hy, p + "mix.right.f.b", l.b_in + l.off_rf, Hr * rk);
      hy_name_rows(hy, p + "mix.right.v", l.w_in, l.off_rv, Hr * rv, D);
      hy_name_vec(hy, p + "mix.right.lower", l.lower, Hr * rk);
      hy_name_vec(hy, p + "mix.right.norm", l.head_norm, rv);
      hy_name_rows(hy, p + "mix.right.o", l.w_o2, 0, D, l.n_o2);
      l.tc_attn = !d.compute_fp32 && dk == dv && (dk == 64 || dk == 128) && H / G <= 8 && c.a_scale > 0.f;
      if (l.tc_attn && (size_t)(H * (dk + dv)) > hy->maxQG) hy->maxQG = H * (dk + dv);
      l.st_rec = st; st += (size_t)(Hr * rv * rk);
      const size_t cc = (size_t)(2 * Hr * rk + Hr * rv);
      if (cc > hy->maxC) hy->maxC = cc;
      if ((size_t)l.n_o > hy->maxO) hy->maxO = l.n_o;
      if ((size_t)l.n_o2 > hy->maxO) hy->maxO = l.n_o2;
      wbytes += ((size_t)l.n_in * D + D * l.n_o + D * l.n_o2) * 2;
      kvpos += (uint64_t)G * (dk + dv) * (d.compute_fp32 ? 4 : 2);
    } else if (c.mixer == XB_MIX_SOFTMAX) {
      XB_TRY(hy_create_softmax(e, i, own, wbytes, kvpos));
    } else if (c.mixer == XB_MIX_LATENT || c.mixer == XB_MIX_GDELTA || c.mixer == XB_MIX_LIGHTNING) {
      XB_TRY(hy_create_mixer(e, i, own, st, wbytes, kvpos));
    } else {
      return xb_fail(1, "layer %d: unknown mixer kind %d", i, c.mixer);
    }
    if (d.gated_residual && l.off_rg >= 0) {   // the mixer's residual gate: rows of the fused input projection
      hy_name_rows(hy, p + "rg1", l.w_in, l.off_rg, D, D);
      hy_name_vec(hy, p + "rg1.b", l.b_in + l.off_rg, D);
    }
    if ((size_t)l.n_in > hy->maxN) hy->maxN = l.n_in;
    if ((size_t)l.n_o > hy->maxK) hy->maxK = l.n_o;
    if ((size_t)l.n_o2 > hy->maxK) hy->maxK = l.n_o2;
    if (c.ff > 0 && c.ff_kind != XB_FF_RELU2) {
      if (branchnorm) { XB_TRY(hy_alloc_t(hy, &l.norm2, nd)); hy_name_vec(hy, p + "norm2", l.norm2, nd); }
      if (sandwich) {   // the feed-forward is a sublayer of its own: norm before and after, optionally the causal filter
        XB_CHECK(own && c.ff_kind == XB_FF_MOE, "layer %d: sandwich blocks take experts with tensors of their own", i);
        XB_TRY(hy_alloc_t(hy, &l.norm2, D)); hy_name_vec(hy, p + "norm2", l.norm2, D);
        XB_TRY(hy_alloc_t(hy, &l.norm2b, D)); hy_name_vec(hy, p + "norm2b", l.norm2b, D);
        if (ct > 0 && !d.ff_unfiltered) {
          XB_TRY(hy_alloc_t(hy, &l.canon2, D * ct)); hy_name(hy, p + "canon2", l.canon2, true, D, ct, ct, 2);
          l.st_canon2 = st; st += (size_t)(ct - 1) * D;
        }
      }
      XB_TRY(hy_create_ff(e, i, own, wbytes));
    } else if (c.ff > 0) {
      XB_CHECK(own && sandwich, "layer %d: the squared-ReLU feed-forward belongs to sandwich blocks with tensors of their own", i);
      const size_t F = c.ff;
      XB_TRY(hy_alloc_t(hy, &l.norm2, D)); hy_name_vec(hy, p + "norm2", l.norm2, D);
      XB_TRY(hy_alloc_t(hy, &l.norm2b, D)); hy_name_vec(hy, p + "norm2b", l.norm2b, D);
      XB_TRY(hy_alloc_t(hy, &l.w_up, F * D)); hy_name_rows(hy, p + "mlp.up", l.w_up, 0, F, D);
      XB_TRY(hy_alloc_t(hy, &l.w_down, D * F)); hy_name_rows(hy, p + "mlp.down", l.w_down, 0, D, F);
      if (ct > 0 && !d.ff_unfiltered) {
        XB_TRY(hy_alloc_t(hy, &l.canon2, D * ct)); hy_name(hy, p + "canon2", l.canon2, true, D, ct, ct, 2);
        l.st_canon2 = st; st += (size_t)(ct - 1) * D;
      }
      if (F > hy->maxN) hy->maxN = F;
      if (F > hy->maxK) hy->maxK = F;
      wbytes += 2 * F * D * 2;
    }
    if (d.side_dim > 0) {
      const size_t sd = d.side_dim;
      XB_TRY(hy_alloc_t(hy, &l.w_sgate, sd * D)); hy_name_rows(hy, p + "side.gate", l.w_sgate, 0, sd, D);
      XB_TRY(hy_alloc_t(hy, &l.w_sproj, D * sd)); hy_name_rows(hy, p + "side.proj", l.w_sproj, 0, D, sd);
      XB_TRY(hy_alloc_t(hy, &l.side_norm, D)); hy_name_vec(hy, p + "side.norm", l.side_norm, D);
      wbytes += 2 * sd * D * 2;
    }
  }
  if (d.bigram_buckets > 0) { hy->st_prev = st; st += 1; }   // a slot's previous token
  hy->state_floats = st;
  if (d.bigram_buckets > 0) {
    XB_TRY(hy_alloc_t(hy, &hy->bigram, (size_t)(d.bigram_buckets + 1) * D));
    hy_name_rows(hy, "bigram", hy->bigram, 0, d.bigram_buckets + 1, D);
    wbytes += D * 2;
  }
  if (d.pos_rows > 0) {
    XB_TRY(hy_alloc_t(hy, &hy->pos_tab, (size_t)d.pos_rows * D));
    hy_name_rows(hy, "pos", hy->pos_tab, 0, d.pos_rows, D);
    wbytes += D * 2;
  }
  // layers that use another layer's tensors: the same device pointers, a cache and state of their own
  for (int i = 0; i < d.n_layers; ++i) {
    HyLayer& l = hy->L[i];
    if (l.owner < 0) continue;
    const HyLayer& o = hy->L[l.owner];
    l.w_in = o.w_in; l.b_in = o.b_in; l.w_o = o.w_o; l.w_up = o.w_up; l.w_down = o.w_down; l.norm1 = o.norm1; l.head_norm = o.head_norm;
    l.w_uk = o.w_uk; l.w_uv = o.w_uv; l.w_d2 = o.w_d2; l.w_router = o.w_router; l.b_up = o.b_up; l.b_down = o.b_down;
    l.lat_norm = o.lat_norm; l.rot_freq = o.rot_freq; l.w0 = o.w0; l.hdecay = o.hdecay; l.canon1 = o.canon1;
  }
  XB_TRY(hy_alloc_t(hy, &hy->embed, (size_t)d.vocab * D)); hy_name_rows(hy, "embed", hy->embed, 0, d.vocab, D);
  if (d.tied_head) hy->head = hy->embed;   // the logits are products with the embedding table itself
  else { XB_TRY(hy_alloc_t(hy, &hy->head, (size_t)d.vocab * D)); hy_name_rows(hy, "head", hy->head, 0, d.vocab, D); }
  XB_TRY(hy_alloc_t(hy, &hy->final_norm, d.norm_scalar ? 1 : D)); hy_name_vec(hy, "final.norm", hy->final_norm, d.norm_scalar ? 1 : D);
  if (d.side_dim > 0) {
    const size_t w = (size_t)d.side_dim * d.n_layers;
    XB_TRY(hy_alloc_t(hy, &hy->side_embed, (size_t)d.vocab * w)); hy_name_rows(hy, "side.embed", hy->side_embed, 0, d.vocab, w);
  }
  wbytes += (size_t)d.vocab * D * 2;
  const size_t as = d.compute_fp32 ? 4 : 2;
  const size_t R = (size_t)(d.max_logit_rows > d.max_seqs ? d.max_logit_rows : d.max_seqs);
  XB_TRY(hy_alloc_t(hy, &hy->x, Tm * D));
  XB_TRY(hy_alloc_t(hy, &hy->hn, Tm * D));
  const size_t ws_min = d.compute_fp32 ? 0 : ((size_t)32 << 20);   // room for the split-K planes of decode-sized batches
  hy->cap_P = Tm * hy->maxN * 4 > ws_min ? Tm * hy->maxN * 4 : ws_min;
  const size_t wm = hy->maxM > D ? hy->maxM : D;
  hy->cap_m = Tm * wm * 4 > ws_min ? Tm * wm * 4 : ws_min;
  XB_TRY(hy_alloc(hy, (void**)&hy->P, hy->cap_P));
  XB_TRY(hy_alloc_t(hy, &hy->c, Tm * hy->maxC));
  XB_TRY(hy_alloc_t(hy, &hy->o, Tm * hy->maxO));
  XB_TRY(hy_alloc(hy, (void**)&hy->m1, hy->cap_m));
  XB_TRY(hy_alloc(hy, (void**)&hy->m2, hy->cap_m));
  XB_TRY(hy_alloc_t(hy, &hy->beta, Tm * hy->maxH));
  XB_TRY(hy_alloc_t(hy, &hy->decay, Tm * hy->maxH));
  XB_TRY(hy_alloc_t(hy, &hy->qk, Tm * hy->maxH));
  XB_TRY(hy_alloc(hy, &hy->a1, Tm * hy->maxK * as));
  XB_TRY(hy_alloc(hy, &hy->a2, Tm * hy->maxK * as));
  XB_TRY(hy_alloc(hy, &hy->head_in, R * D * as));
  if (d.block == XB_BLOCK_PARALLEL) XB_TRY(hy_alloc(hy, &hy->ah, Tm * D * as));
  {
    // the first layer that blends values leaves them for the others, whose value rows must have the same width
    long long first_gv = -1;
    for (HyLayer& l : hy->L) {
      if (l.d.mixer != XB_MIX_SOFTMAX || !l.d.s_vmix) continue;
      const long long gv = (long long)l.d.s_kv_heads * l.d.s_vdim;
      if (first_gv < 0) { first_gv = gv; l.vmode = 1; }
      else { XB_CHECK(gv == first_gv, "layers that blend values carry %lld and %lld of them per token", first_gv, gv); l.vmode = 2; }
    }
    for (size_t i = 0; i < hy->L.size(); ++i) {   // nothing reads the blend factor of the layer whose values the others take
      auto it = hy->names.find("l" + std::to_string(i) + ".mix.vmix");
      if (it != hy->names.end() && hy->L[i].vmode != 2) it->second.optional = true;
    }
  }
  if (hy->maxQA > 0) XB_TRY(hy_alloc_t(hy, &hy->qa, Tm * hy->maxQA));
  if (hy->maxLatR > 0 && !d.compute_fp32) XB_TRY(hy_alloc_t(hy, &hy->lat_part, (size_t)HY_LAT_SPLIT_ROWS * (hy->maxLatR + 2)));
  if (hy->maxE > 0) XB_TRY(hy_alloc_t(hy, &hy->gw, Tm * hy->maxE));
  if (hy->maxGV > 0) XB_TRY(hy_alloc_t(hy, &hy->vfirst, Tm * hy->maxGV));
  hy->cap_head = R * (size_t)d.vocab * 4 > ws_min ? R * (size_t)d.vocab * 4 : ws_min;
  XB_TRY(hy_alloc(hy, (void**)&hy->head_raw, hy->cap_head));
  {
    const char* g = getenv("XB_HY_TC");
    if (g != nullptr && g[0] == '0') hy->use_tc = 0;
    const char* lm = getenv("XB_HY_LAT_MMA");
    if (lm != nullptr) hy->use_lat_mma = atoi(lm);   // 0: off; 1: by the step's shape; 4: always the four-warp unsplit form; 2: always key shares
    const char* ta = getenv("XB_HY_TC_ATTN");
    if (ta != nullptr && ta[0] == '0') hy->use_tc_attn = 0;
    const char* ga = getenv("XB_HY_GATHER");
    if (ga != nullptr && ga[0] == '0') hy->use_gather = 0;
    const char* fr = getenv("XB_HY_FUSE_ROUTER");
    if (fr != nullptr && fr[0] == '0') hy->fuse_router = 0;
    const char* ps = getenv("XB_HY_P_SPLIT");
    if (ps != nullptr && ps[0] == '0') hy->p_split = 0;
    const char* lp = getenv("XB_HY_LPC");
    if (lp != nullptr && (atoi(lp) == 4 || atoi(lp) == 8 || atoi(lp) == 16)) hy->recur_lpc = atoi(lp);
  }
  XB_TRY(hy_alloc_t(hy, &hy->d_rows, R));
  if (hy->maxQG > 0) {
    XB_TRY(hy_alloc_t(hy, &hy->qg, Tm * hy->maxQG));
    std::vector<int> ones((size_t)d.max_seqs, 1);
    XB_TRY(hy_alloc_t(hy, &hy->d_ones, (size_t)d.max_seqs));
    XB_CUDA(cudaMemcpy(hy->d_ones, ones.data(), ones.size() * sizeof(int), cudaMemcpyHostToDevice));
  }
  XB_TRY(dmalloc((void**)&e->logits, R * (size_t)d.vocab * sizeof(float)));
  e->c.weight_bytes = wbytes;
  e->c.kv_bytes_per_pos = kvpos;
  return 0;
}

// ----------------------------------------------------------------------------- weights
static int hy_store(xb_engine* e, const std::string& name, const void* src, int dt, const long long* shape, int ndim, bool src_on_device) {
  HyModel* hy = e->hy;
  auto it = hy->names.find(name);
  if (it == hy->names.end()) return xb_fail(1, "tensor %s is not part of this model", name.c_str());
  const HyTarget& t = it->second;
  XB_CHECK(dt >= 0 && dt <= 2, "tensor %s: unsupported element type", name.c_str());
  long long numel = 1;
  for (int i = 0; i < ndim; ++i) numel *= shape[i];
  bool ok = numel == t.rows * t.cols && (ndim == t.ndim || numel == 1);   // a single number may come without a shape
  if (ok && ndim == 2) ok = shape[0] == t.rows && shape[1] == t.cols;
  if (!ok) {
    std::string got;
    for (int i = 0; i < ndim; ++i) got += (i ? "x" : "") + std::to_string(shape[i]);
    return xb_fail(1, "tensor %s has shape %s, this model wants %lldx%lld", name.c_str(), got.c_str(), t.rows, t.cols);
  }
  const size_t bytes = (size_t)numel * (dt == 2 ? 4 : 2);
  const void* dsrc = src;
  void* staging = nullptr;
  if (!src_on_device) {
    XB_TRY(dmalloc(&staging, bytes));
    XB_CUDA(cudaMemcpy(staging, src, bytes, cudaMemcpyHostToDevice));
    dsrc = staging;
  }
  const unsigned blocks = (unsigned)((numel + 255) / 256);
  if (t.f32) hy_load_convert_kernel<float><<<blocks, 256>>>(dsrc, dt, t.rows, t.cols, (float*)t.dst, t.ld);
  else hy_load_convert_kernel<bf16><<<blocks, 256>>>(dsrc, dt, t.rows, t.cols, (bf16*)t.dst, t.ld);
  XB_CUDA(cudaGetLastError());
  XB_CUDA(cudaDeviceSynchronize());
  if (staging) cudaFree(staging);
  hy->loaded.insert(name);
  hy->finalized = false;
  return 0;
}

// bf16 serving: once every tensor is in, each matrix the tcgen05 Linear can take (K a multiple of 8, at least one
// 64-wide k block and 16 rows) gets its tile-major copy.  Runs before the first forward (never inside a capture).
static int hy_tile(bf16** dst, const bf16* src, size_t rows, size_t K) {
  if (*dst != nullptr || K % 8 != 0 || K < 64 || rows < 16) return 0;
  XB_TRY(alloc_tiled(dst, rows, K));
  return store_tiled(*dst, src, 0, rows, K);
}
static int hy_n_missing(const HyModel* hy) {
  int n = 0;
  for (const auto& kv : hy->names) n += (!kv.second.optional && !hy->loaded.count(kv.first)) ? 1 : 0;
  return n;
}
static int hy_finalize(xb_engine* e) {
  HyModel* hy = e->hy;
  if (hy->finalized) return 0;
  hy->finalized = true;
  hy->plans.clear();
  if (hy->d.compute_fp32 || !hy->use_tc || hy_n_missing(hy) > 0) return 0;
  const size_t D = hy->d.dim;
  auto retile = [&](bf16** dst, const bf16* src, size_t rows, size_t K) -> int {
    if (*dst != nullptr) { cudaFree(*dst); *dst = nullptr; }
    return src != nullptr ? hy_tile(dst, src, rows, K) : 0;
  };
  for (HyLayer& l : hy->L) {
    if (l.owner >= 0) continue;
    const size_t n_up = l.n_up > 0 ? l.n_up : l.d.ff, n_dn = l.n_dn > 0 ? l.n_dn : l.d.ff;
    XB_TRY(retile(&l.t_in, l.w_in, l.n_in, D));
    XB_TRY(retile(&l.t_o, l.w_o, D, l.n_o));
    XB_TRY(retile(&l.t_o2, l.w_o2, D, l.n_o2));
    XB_TRY(retile(&l.t_up, l.w_up, n_up, D));
    XB_TRY(retile(&l.t_down, l.w_down, D, n_dn));
    XB_TRY(retile(&l.t_sgate, l.w_sgate, hy->d.side_dim, D));
    XB_TRY(retile(&l.t_sproj, l.w_sproj, D, hy->d.side_dim));
    XB_TRY(retile(&l.t_d2, l.w_d2, (size_t)l.d.m_heads * l.d.m_dim, l.d.m_rank));
  }
  for (HyLayer& l : hy->L) {
    if (l.owner < 0) continue;
    const HyLayer& o = hy->L[l.owner];
    l.t_in = o.t_in; l.t_o = o.t_o; l.t_up = o.t_up; l.t_down = o.t_down; l.t_d2 = o.t_d2;
  }
  XB_TRY(retile(&hy->t_head, hy->head, hy->d.vocab, D));
  return 0;
}

static int hy_load_file(xb_engine* e, const char* path, const std::vector<StEntry>& entries, const uint8_t* data, size_t data_size,
                        int* n_tensors, uint64_t* n_bytes) {
  int count = 0;
  uint64_t total = 0;
  for (const StEntry& en : entries) {
    if (e->hy->names.find(en.name) == e->hy->names.end()) continue;
    const int dt = st_dtype_code(en.dtype);
    XB_CHECK(dt >= 0, "%s: tensor %s has unsupported dtype %s (BF16, F16, F32)", path, en.name.c_str(), en.dtype.c_str());
    long long numel = 1;
    for (long long v : en.shape) numel *= v;
    XB_CHECK(en.end <= data_size && en.end - en.begin == (size_t)numel * st_dtype_size(dt), "%s: tensor %s: size and shape disagree",
             path, en.name.c_str());
    XB_TRY(hy_store(e, en.name, data + en.begin, dt, en.shape.data(), (int)en.shape.size(), false));
    ++count;
    total += en.end - en.begin;
  }
  if (n_tensors) *n_tensors = count;
  if (n_bytes) *n_bytes = total;
  return 0;
}

static int hy_missing(xb_engine* e, char* buf, size_t buflen, int* n_missing) {
  std::string out;
  int n = 0;
  for (const auto& kv : e->hy->names) {
    if (kv.second.optional || e->hy->loaded.count(kv.first)) continue;
    ++n;
    if (out.size() < 900) out += kv.first + "; ";
  }
  *n_missing = n;
  if (buf != nullptr && buflen > 0) {
    strncpy(buf, out.c_str(), buflen - 1);
    buf[buflen - 1] = 0;
  }
  return 0;
}

// ----------------------------------------------------------------------------- slots: KV pools + state
static int hy_reserve(xb_engine* e) {
  HyModel* hy = e->hy;
  const size_t es = hy->d.compute_fp32 ? 4 : 2;
  for (HyLayer& l : hy->L) {
    cudaFree(l.k_pool); cudaFree(l.v_pool);
    l.k_pool = l.v_pool = nullptr;
    if (l.d.mixer == XB_MIX_LATENT) {   // one pool: a row holds the latent (key and value at once) and the rotated key part
      const size_t kb = (size_t)e->n_pages * e->page_tokens * (l.d.m_kv_rank + l.d.m_rot_dim) * es;
      XB_TRY(dmalloc(&l.k_pool, kb));
      XB_CUDA(cudaMemset(l.k_pool, 0, kb));
      continue;
    }
    if (l.d.mixer == XB_MIX_SOFTMAX) {   // keys [page][G][token][dk]; values the same way, or [page][token][G * dv] (v_all)
      const size_t kb = (size_t)e->n_pages * l.d.s_kv_heads * e->page_tokens * l.d.s_dim * es;
      const size_t vb = (size_t)e->n_pages * l.d.s_kv_heads * e->page_tokens * l.d.s_vdim * es;
      XB_TRY(dmalloc(&l.k_pool, kb));
      XB_TRY(dmalloc(&l.v_pool, vb));
      XB_CUDA(cudaMemset(l.k_pool, 0, kb));
      XB_CUDA(cudaMemset(l.v_pool, 0, vb));
      if (l.tc_attn) {
        const long long G = l.d.s_kv_heads, pool_rows = (long long)e->n_pages * G * e->page_tokens;
        const int box_rows = e->page_tokens < 64 ? e->page_tokens : 64;
        XB_TRY(xb_make_tmap(&l.tmK, l.k_pool, pool_rows, l.d.s_dim, l.d.s_dim, box_rows));
        if (l.v_all) XB_TRY(xb_make_tmap(&l.tmV, l.v_pool, pool_rows / G, G * l.d.s_vdim, G * l.d.s_vdim, box_rows));
        else XB_TRY(xb_make_tmap(&l.tmV, l.v_pool, pool_rows, l.d.s_vdim, l.d.s_vdim, box_rows));
      }
      continue;
    }
    if (l.d.mixer != XB_MIX_PARALLEL) continue;
    const size_t kb = (size_t)e->n_pages * l.d.a_kv_heads * e->page_tokens * l.d.a_dim * es;
    const size_t vb = (size_t)e->n_pages * l.d.a_kv_heads * e->page_tokens * l.d.a_vdim * es;
    XB_TRY(dmalloc(&l.k_pool, kb));
    XB_TRY(dmalloc(&l.v_pool, vb));
    XB_CUDA(cudaMemset(l.k_pool, 0, kb));
    XB_CUDA(cudaMemset(l.v_pool, 0, vb));
    if (l.tc_attn) {
      const long long pool_rows = (long long)e->n_pages * l.d.a_kv_heads * e->page_tokens;
      const int box_rows = e->page_tokens < 64 ? e->page_tokens : 64;
      XB_TRY(xb_make_tmap(&l.tmK, l.k_pool, pool_rows, l.d.a_dim, l.d.a_dim, box_rows));
      XB_TRY(xb_make_tmap(&l.tmV, l.v_pool, pool_rows, l.d.a_vdim, l.d.a_vdim, box_rows));
    }
  }
  cudaFree(hy->state);
  hy->state = nullptr;
  const size_t sb = (size_t)e->n_slots * (hy->state_floats ? hy->state_floats : 1) * sizeof(float);
  XB_TRY(dmalloc((void**)&hy->state, sb));
  XB_CUDA(cudaMemset(hy->state, 0, sb));
  return 0;
}

// Query tiles of the tcgen05 attention hold 128 rows = tokens x (query heads per key head); one tile table serves every
// attention layer, so it is cut for the largest group among them.
static int hy_tile_tokens(const xb_hybrid_desc& d, const xb_hybrid_layer* layers) {
  int tt = 128;
  for (int i = 0; i < d.n_layers; ++i) {
    const xb_hybrid_layer& c = layers[i];
    int group = 0;
    if (c.mixer == XB_MIX_PARALLEL && c.a_kv_heads > 0 && c.a_heads % c.a_kv_heads == 0) group = c.a_heads / c.a_kv_heads;
    if (c.mixer == XB_MIX_SOFTMAX && c.s_kv_heads > 0 && c.s_heads % c.s_kv_heads == 0) group = c.s_heads / c.s_kv_heads;
    if (group >= 1 && group <= 8 && 128 / group < tt) tt = 128 / group;
  }
  return tt;
}

// ----------------------------------------------------------------------------- forward
template <typename... KArgs, typename... Args>
static int hy_launch(xb_engine* e, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  if (e->use_pdl && e->hy->pdl_now) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  XB_CUDA(cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...));
  e->c.launches++;
  return 0;
}

static LinOut hy_plain(const float* f, long long ld) {
  LinOut o;
  o.f = f; o.h = nullptr; o.si = SplitInfo{0, 0, 0}; o.plane = 0; o.ld = ld; o.bias = nullptr;
  return o;
}
static LinOut hy_none() { return hy_plain(nullptr, 0); }

// The engine's tcgen05 Linear on a tile-major weight copy: decode-sized batches leave fp32 split-K planes, larger ones a
// bf16 matrix; either way the consumer reads through LinOut (bias added on read).  false: not applicable here.
static bool hy_tc_linear(xb_engine* e, const void* x, long long ldx, const bf16* wt, const float* bias, int T, int N, int K, void* out,
                         size_t cap, cudaStream_t st, LinOut* y, int* rc) {
  HyModel* hy = e->hy;
  *rc = 0;
  if (wt == nullptr || ldx % 8 != 0) return false;
  const auto key = std::make_tuple((const void*)wt, x, (const void*)out, T);
  auto it = hy->plans.find(key);
  if (it == hy->plans.end()) {
    GemmPlan p;
    const int sms = (T <= 128 && e->reserved_sms > 0 && e->reserved_sms < e->num_sms) ? e->num_sms - e->reserved_sms : e->num_sms;
    if ((*rc = xb_gemm_plan(&p, (const bf16*)x, ldx, wt, 1, T, N, K, out, N, nullptr, 0, sms, 0)) != 0) return true;
    const size_t need = p.args.mode == XB_GEMM_SKINNY ? (size_t)p.split.splits * T * N * 4 : (size_t)T * N * 2;
    if (need > cap) return false;
    it = hy->plans.emplace(key, p).first;
  }
  const GemmPlan& p = it->second;
  if ((*rc = run_gemm(e, p, st)) != 0) return true;
  LAUNCH_COUNT(e);
  LinOut o;
  o.ld = N; o.bias = bias; o.plane = (long long)T * N;
  if (p.args.mode == XB_GEMM_SKINNY) { o.f = (const float*)out; o.h = nullptr; o.si = p.split; }
  else { o.f = nullptr; o.h = (const bf16*)out; o.si = SplitInfo{0, 0, 0}; }
  *y = o;
  return true;
}

// y[T, N] = x[T, K] w^T + bias into `out` (`cap` bytes).  wt: the weight's tile-major copy or nullptr.
template <typename AT>
static int hy_linear(xb_engine* e, const void* x, long long ldx, const bf16* w, const bf16* wt, const float* bias, int T, int N, int K,
                     float* out, size_t cap, cudaStream_t st, LinOut* y) {
  if (std::is_same<AT, bf16>::value) {
    int rc = 0;
    if (hy_tc_linear(e, x, ldx, wt, bias, T, N, K, out, cap, st, y, &rc)) return rc;
  }
  const AT* xa = reinterpret_cast<const AT*>(x);
  if (T <= HY_SMALL_T)
    XB_TRY(hy_launch(e, hy_linear_small_kernel<AT>, dim3((N + 7) / 8), dim3(256), 0, st, xa, ldx, w, bias, out, (long long)N, T, N, K));
  else
    XB_TRY(hy_launch(e, hy_linear_tiled_kernel<AT>, dim3((N + 63) / 64, (T + 63) / 64), dim3(256), 0, st, xa, ldx, w, bias, out,
                     (long long)N, T, N, K));
  *y = hy_plain(out, N);
  return 0;
}

// one recurrence launch.  Lanes per state column: the fewest of 4, 8, 16 that still give two blocks per SM (one long
// prompt wants many short chains, a batch of sequences few shuffles); then the fewest chunks per lane that cover the key dim.
template <int LPC, int MODE>
static int hy_recur_l(xb_engine* e, const RecurIn& in, float* state, long long ss, float* o, long long ldo, const BatchMeta& m,
                      int n_seqs, int H, int dk, int dv, cudaStream_t st) {
  constexpr int COLS = 128 / LPC;
  const dim3 grid(n_seqs, H, (dv + COLS - 1) / COLS);
#define HY_RECUR_CASE(NCH)                                                                                               \
  if (dk <= 4 * LPC * NCH) {                                                                                             \
    const size_t smem = (size_t)2 * HY_TS * (hy_rec_vectors(MODE) * 4 * LPC * NCH + COLS + 4) * sizeof(float);           \
    if (smem > 48 * 1024) XB_SMEM_ATTR_ONCE((hy_recur_kernel<NCH, LPC, MODE>), smem);                                    \
    return hy_launch(e, hy_recur_kernel<NCH, LPC, MODE>, grid, dim3(128), smem, st, in, state, ss, o, ldo, m, H, dk, dv); \
  }
  HY_RECUR_CASE(1)
  HY_RECUR_CASE(2)
  HY_RECUR_CASE(4)
  if constexpr (LPC <= 8) { HY_RECUR_CASE(8) }
  if constexpr (LPC <= 4) { HY_RECUR_CASE(16) }
#undef HY_RECUR_CASE
  return xb_fail(1, "recurrent key dim %d exceeds %d", dk, HY_MAX_KDIM);
}
template <int MODE>
static int hy_recur(xb_engine* e, const RecurIn& in, float* state, long long ss, float* o, long long ldo, const BatchMeta& m, int n_seqs,
                    int H, int dk, int dv, cudaStream_t st) {
  int lpc = e->hy->recur_lpc;
  if (lpc == 0) {
    const long long want = 2LL * e->num_sms;
    lpc = 16;
    if ((long long)n_seqs * H * ((dv + 31) / 32) >= want) lpc = 4;
    else if ((long long)n_seqs * H * ((dv + 15) / 16) >= want) lpc = 8;
  }
  if (lpc == 4) return hy_recur_l<4, MODE>(e, in, state, ss, o, ldo, m, n_seqs, H, dk, dv, st);
  if (lpc == 8) return hy_recur_l<8, MODE>(e, in, state, ss, o, ldo, m, n_seqs, H, dk, dv, st);
  return hy_recur_l<16, MODE>(e, in, state, ss, o, ldo, m, n_seqs, H, dk, dv, st);
}

// causal per-channel filter over T rows (+ the slots' new tails): tap counts up to 4 through the tiled kernel, which in a
// step of single tokens (no_span) also writes the tails; anything else through the general pair of kernels
template <typename OT>
static int hy_filter(xb_engine* e, int T, int n_seqs, bool no_span, const LinOut& in, int col0, int C, int taps, const float* w, float* tail,
                     const BatchMeta& m, int identity, int act_silu, OT* out, long long ld_out, cudaStream_t st) {
  const long long SS = (long long)e->hy->state_floats;
  bool tail_done = false;
  const bool few = T <= 64;   // a block per row instead of 16 rows per thread
  const dim3 tg(few ? T : (T + 15) / 16, (C + 255) / 256);
  const int wt = no_span ? 1 : 0;
  switch (taps) {
#define HY_TAPS_CASE(N)                                                                                                          \
  case N:                                                                                                                        \
    if (few)                                                                                                                     \
      XB_TRY(hy_launch(e, hy_taps_tile_kernel<OT, N, 1>, tg, dim3(256), 0, st, in, col0, C, w, tail, SS, m, identity, act_silu, wt, out, \
                       ld_out, T));                                                                                              \
    else                                                                                                                         \
      XB_TRY(hy_launch(e, hy_taps_tile_kernel<OT, N, 16>, tg, dim3(256), 0, st, in, col0, C, w, tail, SS, m, identity, act_silu, wt, out, \
                       ld_out, T));                                                                                              \
    tail_done = no_span;                                                                                                         \
    break;
    HY_TAPS_CASE(1)
    HY_TAPS_CASE(2)
    HY_TAPS_CASE(3)
    HY_TAPS_CASE(4)
#undef HY_TAPS_CASE
    default:
      XB_TRY(hy_launch(e, hy_taps_kernel<OT>, dim3(T, (C + 255) / 256), dim3(256), 0, st, in, col0, C, taps, w, (const float*)tail, SS, m,
                       identity, act_silu, out, ld_out));
  }
  if (taps > 1 && !tail_done)
    XB_TRY(hy_launch(e, hy_tail_update_kernel, dim3(n_seqs, (C + 255) / 256), dim3(256), 0, st, in, col0, C, taps, tail, SS, m));
  return 0;
}

struct HyAttnIn {
  const bf16* q;             // q rows, pitch io.ldq
  AttIo io;
  const int *tile_start, *tile_len;
  int n_tiles;
};
template <int HD, int GRP>
static int hy_attn_tc_g(xb_engine* e, const HyLayer& l, const BatchMeta& m, const HyAttnIn& in, bf16* out, cudaStream_t st) {
  using Cfg = AttTcCfg<HD>;
  const xb_hybrid_layer& c = l.d;
  XB_SMEM_ATTR_ONCE((xb_attn_prefill_tc_kernel<HD, GRP>), Cfg::SMEM_BYTES);
  const AttMask mk{c.a_window, c.a_keep_first};
  e->c.tc_attention++;
  return hy_launch(e, xb_attn_prefill_tc_kernel<HD, GRP>, dim3(in.n_tiles, c.a_kv_heads), dim3(192), Cfg::SMEM_BYTES, st, l.tmK, l.tmV,
                   in.q, m, in.tile_start, in.tile_len, out, c.a_heads, c.a_kv_heads, c.a_scale * 1.4426950408889634f, mk, in.io);
}
template <int HD>
static int hy_attn_tc(xb_engine* e, const HyLayer& l, const BatchMeta& m, const HyAttnIn& in, bf16* out, cudaStream_t st) {
  switch (l.d.a_heads / l.d.a_kv_heads) {
    case 1: return hy_attn_tc_g<HD, 1>(e, l, m, in, out, st);
    case 2: return hy_attn_tc_g<HD, 2>(e, l, m, in, out, st);
    case 3: return hy_attn_tc_g<HD, 3>(e, l, m, in, out, st);
    case 4: return hy_attn_tc_g<HD, 4>(e, l, m, in, out, st);
    case 5: return hy_attn_tc_g<HD, 5>(e, l, m, in, out, st);
    case 6: return hy_attn_tc_g<HD, 6>(e, l, m, in, out, st);
    case 7: return hy_attn_tc_g<HD, 7>(e, l, m, in, out, st);
    case 8: return hy_attn_tc_g<HD, 8>(e, l, m, in, out, st);
  }
  return xb_fail(1, "no tcgen05 attention for %d query heads per key head", l.d.a_heads / l.d.a_kv_heads);
}

// the tcgen05 prompt attention for any layer kind: H query / KV key heads, grid z blocks per (tile, key head)
template <int HD, int GRP>
static int hy_attn_tc_any_g(xb_engine* e, const HyLayer& l, const BatchMeta& m, const HyAttnIn& in, bf16* out, int H, int KV, float scale, int gz,
                            cudaStream_t st) {
  using Cfg = AttTcCfg<HD>;
  XB_SMEM_ATTR_ONCE((xb_attn_prefill_tc_kernel<HD, GRP, true>), Cfg::SMEM_BYTES);
  e->c.tc_attention++;
  return hy_launch(e, xb_attn_prefill_tc_kernel<HD, GRP, true>, dim3(in.n_tiles, KV, gz), dim3(192), Cfg::SMEM_BYTES, st, l.tmK, l.tmV, in.q, m,
                   in.tile_start, in.tile_len, out, H, KV, scale * 1.4426950408889634f, AttMask{0, 0}, in.io);
}
template <int HD>
static int hy_attn_tc_any(xb_engine* e, const HyLayer& l, const BatchMeta& m, const HyAttnIn& in, bf16* out, int H, int KV, float scale, int gz,
                          cudaStream_t st) {
  switch (H / KV) {
    case 1: return hy_attn_tc_any_g<HD, 1>(e, l, m, in, out, H, KV, scale, gz, st);
    case 2: return hy_attn_tc_any_g<HD, 2>(e, l, m, in, out, H, KV, scale, gz, st);
    case 3: return hy_attn_tc_any_g<HD, 3>(e, l, m, in, out, H, KV, scale, gz, st);
    case 4: return hy_attn_tc_any_g<HD, 4>(e, l, m, in, out, H, KV, scale, gz, st);
    case 5: return hy_attn_tc_any_g<HD, 5>(e, l, m, in, out, H, KV, scale, gz, st);
    case 6: return hy_attn_tc_any_g<HD, 6>(e, l, m, in, out, H, KV, scale, gz, st);
    case 7: return hy_attn_tc_any_g<HD, 7>(e, l, m, in, out, H, KV, scale, gz, st);
    case 8: return hy_attn_tc_any_g<HD, 8>(e, l, m, in, out, H, KV, scale, gz, st);
  }
  return xb_fail(1, "no tcgen05 attention for %d query heads per key head", H / KV);
}

// A step of single tokens through the engine's split-key decode attention (mma.sync over TMA-staged tiles, the splits of a
// (token, key head) merged inside a thread-block cluster), with the sink / cap / wide-value options of the layer.
template <int HD, int GRP>
static int hy_attn_dec_g(xb_engine* e, const HyLayer& l, const BatchMeta& m, int T, const bf16* q, bf16* out, int H, int KV, float scale,
                         int n_splits, const AttDecOpt& opt, cudaStream_t st) {
  constexpr int NST = 3;
  using Cfg = AttDecCfg<HD, GRP, NST>;
  auto kern = xb_attn_decode_mma_kernel<HD, GRP, NST, false>;
  XB_SMEM_ATTR_ONCE(kern, Cfg::SMEM_BYTES);
  const dim3 grid(T, opt.v_wide ? KV * KV : KV, n_splits);
  return launch_kc(e, kern, grid, dim3(160), Cfg::SMEM_BYTES, st, dim3(1, 1, n_splits), l.tmK, l.tmV, q, m, (float*)nullptr, (float*)nullptr, out,
                   H, KV, n_splits, scale * 1.4426950408889634f, QkvFin{}, n_splits > 1 ? 1 : 0, opt);
}
template <int HD>
static int hy_attn_dec(xb_engine* e, const HyLayer& l, const BatchMeta& m, int T, const bf16* q, bf16* out, int H, int KV, float scale,
                       int n_splits, const AttDecOpt& opt, cudaStream_t st) {
  switch (H / KV) {
    case 1: return hy_attn_dec_g<HD, 1>(e, l, m, T, q, out, H, KV, scale, n_splits, opt, st);
    case 2: return hy_attn_dec_g<HD, 2>(e, l, m, T, q, out, H, KV, scale, n_splits, opt, st);
    case 3: return hy_attn_dec_g<HD, 3>(e, l, m, T, q, out, H, KV, scale, n_splits, opt, st);
    case 4: return hy_attn_dec_g<HD, 4>(e, l, m, T, q, out, H, KV, scale, n_splits, opt, st);
    case 5: return hy_attn_dec_g<HD, 5>(e, l, m, T, q, out, H, KV, scale, n_splits, opt, st);
    case 6: return hy_attn_dec_g<HD, 6>(e, l, m, T, q, out, H, KV, scale, n_splits, opt, st);
    case 7: return hy_attn_dec_g<HD, 7>(e, l, m, T, q, out, H, KV, scale, n_splits, opt, st);
    case 8: return hy_attn_dec_g<HD, 8>(e, l, m, T, q, out, H, KV, scale, n_splits, opt, st);
  }
  return xb_fail(1, "no decode attention for %d query heads per key head", H / KV);
}

template <typename AT>
static int hy_row_op_launch(xb_engine* e, int T, const RowOpArgs& a, cudaStream_t st);
// sandwich blocks: x += residual_mult * norm(s1 m1 + s2 m2) * weight, then the next reader's norm into hn (and, as a Linear
// input, into ha when given).  Weights are offsets from one or plain, norms whole-row or grouped, as the model says.
template <typename AT>
static int hy_row_op(xb_engine* e, int T, LinOut m1, float s1, LinOut m2, float s2, const float* bw, float bw_one, const float* nw,
                     void* xa, cudaStream_t st, void* ha = nullptr) {
  HyModel* hy = e->hy;
  RowOpArgs a;
  a.x = hy->x; a.m1 = m1; a.m2 = m2; a.s1 = s1; a.s2 = s2; a.bw = bw; a.bw_one = hy->d.norm_plain ? 0.f : bw_one; a.nw = nw; a.hn = hy->hn; a.xa = xa;
  a.eps = hy->d.norm_eps; a.D = hy->d.dim;
  a.m3 = hy_none(); a.ha = ha; a.plain_add = 0; a.nw_mode = hy->d.norm_plain ? 1 : 0;
  a.groups = hy->d.norm_groups > 1 ? hy->d.norm_groups : 1;
  a.res_mult = hy->d.residual_mult != 0.f ? hy->d.residual_mult : 1.f;
  a.ext = (hy->d.norm_plain || a.groups > 1 || a.res_mult != 1.f || ha != nullptr) ? 1 : 0;
  return hy_row_op_launch<AT>(e, T, a, st);
}
template <typename AT>
static int hy_row_op_launch(xb_engine* e, int T, const RowOpArgs& a, cudaStream_t st) {
  HyModel* hy = e->hy;
  const bool few = T <= 64 && hy->d.dim >= 1024;   // decode-sized batches: few rows, so more threads per row keep more loads in flight
  // prompts whose branch is one bf16 matrix out of the tensor-core Linear: eight channels per thread
  if (!few && !a.plain_add && a.m1.h != nullptr && a.m1.bias == nullptr && a.m1.ld % 8 == 0 && a.m2.f == nullptr && a.m2.h == nullptr &&
      hy->d.dim % 8 == 0)
    return hy_launch(e, hy_row_op_vec_kernel<AT>, dim3(T), dim3(256), (size_t)hy->d.dim * sizeof(float), st, a);
  if (a.ext && !a.plain_add) {   // grouped norms, residual multiplier, plain weights, the norm as a Linear input
    if (few) return hy_launch(e, hy_row_op_ext_kernel<AT, 1024>, dim3(T), dim3(1024), (size_t)hy->d.dim * sizeof(float), st, a);
    return hy_launch(e, hy_row_op_ext_kernel<AT, 256>, dim3(T), dim3(256), (size_t)hy->d.dim * sizeof(float), st, a);
  }
  if (few) return hy_launch(e, hy_row_op_kernel<AT, 1024>, dim3(T), dim3(1024), (size_t)hy->d.dim * sizeof(float), st, a);
  return hy_launch(e, hy_row_op_kernel<AT, 256>, dim3(T), dim3(256), (size_t)hy->d.dim * sizeof(float), st, a);
}

// what a sublayer reads: the normed stream plus its causal filter, as a Linear input; then the slot's new tail
template <typename AT>
static int hy_sublayer_input(xb_engine* e, int T, int n_seqs, bool no_span, const float* w, size_t st_off, const BatchMeta& m, cudaStream_t st) {
  HyModel* hy = e->hy;
  const int D = hy->d.dim;
  return hy_filter<AT>(e, T, n_seqs, no_span, hy_plain(hy->hn, D), 0, D, hy->d.taps, w, hy->state + st_off, m, 1, 0,
                       reinterpret_cast<AT*>(hy->a1), (long long)D, st);
}

// Latent attention through hy_latent_attn_mma_kernel.  0: launched; 1: not applicable (shared memory); < 0: -error.
template <int WARPS, int DVC, int LOADW>
static int hy_latent_mma_launch(xb_engine* e, const HyLayer& l, const BatchMeta& m, int T, int n_splits, cudaStream_t st) {
  HyModel* hy = e->hy;
  const xb_hybrid_layer& c = l.d;
  const int H = c.m_heads, R = c.m_kv_rank, W = R + c.m_rot_dim, NR = T * H;
  const int pitch = ((W + 15) & ~15) + 8;
  const size_t smem = (size_t)(16 * WARPS + 2 * HY_LAT_KEYS) * pitch * sizeof(bf16);
  if (smem > 200 * 1024) return 1;
  if (smem > 48 * 1024) {
    static size_t granted[XB_MAX_DEVICES] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= XB_MAX_DEVICES) return 1;
    if (granted[dev] < smem) {
      if (cudaFuncSetAttribute(hy_latent_attn_mma_kernel<WARPS, DVC, LOADW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) return 1;
      granted[dev] = 200 * 1024;
    }
  }
  const dim3 grid((NR + 16 * WARPS - 1) / (16 * WARPS), n_splits, (R + DVC - 1) / DVC);
  if (hy_launch(e, hy_latent_attn_mma_kernel<WARPS, DVC, LOADW>, grid, dim3(32 * LOADW), smem, st, (const float*)hy->qa, (const bf16*)l.k_pool, m, T, H, W,
                R, c.m_scale * 1.4426950408889634f, n_splits, hy->lat_part, hy->o, (long long)H * R) != 0)
    return -1;
  if (n_splits > 1 &&
      hy_launch(e, hy_latent_merge_kernel, dim3(NR), dim3(128), 0, st, (const float*)hy->lat_part, n_splits, NR, H, R, hy->o, (long long)H * R) != 0)
    return -1;
  return 0;
}
static int hy_latent_mma(xb_engine* e, const HyLayer& l, const BatchMeta& m, int T, cudaStream_t st) {
  const int R = l.d.m_kv_rank, NR = T * l.d.m_heads;
  const int tiles4 = (NR + 63) / 64, tiles1 = (NR + 15) / 16;
  const int mode = e->hy->use_lat_mma;
  if (mode == 4 || (mode != 2 && tiles4 >= e->num_sms / 2)) {   // prompts: four warps of rows per block, every block walks its keys alone
    return R <= 128 ? hy_latent_mma_launch<4, 128, 4>(e, l, m, T, 1, st) : hy_latent_mma_launch<4, 256, 4>(e, l, m, T, 1, st);
  }
  int ns = HY_LAT_SPLIT_ROWS / 16 / tiles1;
  ns = ns < 1 ? 1 : (ns > 64 ? 64 : ns);
  return R <= 128 ? hy_latent_mma_launch<1, 128, 4>(e, l, m, T, ns, st) : hy_latent_mma_launch<1, 256, 4>(e, l, m, T, ns, st);
}

// Latent attention of one layer: P = [q | down-projection (| other rows)] of the step's rows -> a1 = what the output
// projection reads.  The cache row is made and appended, the queries are folded into the cache's space, the attention
// runs over the cached latents, and the read-out goes through the value up-projection.
template <typename AT>
static int hy_latent_mixer(xb_engine* e, const HyLayer& l, int T, const LinOut& P, const BatchMeta& m, cudaStream_t st) {
  HyModel* hy = e->hy;
  const xb_hybrid_layer& c = l.d;
  const xb_hybrid_desc& d = hy->d;
  typedef typename std::conditional<std::is_same<AT, float>::value, float, bf16>::type KT;
  AT* a1 = reinterpret_cast<AT*>(hy->a1);
  const int H = c.m_heads, n = c.m_dim;
  const int dr = c.m_rot_dim, dv = c.m_vdim, R = c.m_kv_rank, W = R + dr;
  XB_TRY(hy_launch(e, hy_latent_prep_kernel<KT>, dim3(T), dim3(256), 0, st, P, l.off_q, l.off_dkv, H, n, dr, R, c.m_rot_dims,
                   (const float*)l.rot_freq, (const float*)l.lat_norm, d.norm_eps, (KT*)l.k_pool, m, hy->qa));
  const size_t mm1 = (size_t)HY_MM_ROWS * n * sizeof(float), mm2 = (size_t)HY_MM_ROWS * R * sizeof(float);
  XB_TRY(hy_launch(e, hy_head_mm_t_kernel, dim3((T + HY_MM_ROWS - 1) / HY_MM_ROWS, H), dim3(256), mm1, st, P, l.off_q, n + dr,
                   (const bf16*)l.w_uk, hy->qa, (long long)H * W, W, T, n, R));
  // bf16 serving at sizes the tensor-core tiles take: rows = (token, head) pairs over shared key tiles; steps of few
  // rows split every sequence's keys over blocks and merge
  bool done = false;
  if (std::is_same<AT, bf16>::value && hy->use_lat_mma && W % 8 == 0 && R % 16 == 0) {
    int rc = hy_latent_mma(e, l, m, T, st);
    if (rc < 0) return -rc;
    done = rc == 0;
  }
  if (!done) {
    const int aw = 16;   // causal: every earlier key is visible
    const size_t asm_bytes = (size_t)(((W + 3) & ~3) + aw * (2 + R)) * sizeof(float);
    const LinOut Q = hy_plain(hy->qa, (long long)H * W);
    const int far = 1 << 30;
    if (R <= 256)
      XB_TRY(hy_launch(e, hy_attn_window_kernel<KT, float, 8>, dim3(T, H), dim3(32 * aw), asm_bytes, st, Q, 0, -1, (const KT*)l.k_pool,
                       (const KT*)l.k_pool, m, H, 1, W, R, W, W, far, 0, c.m_scale, 1.0f, hy->o, (long long)H * R, AttnOpt{nullptr, 0.f, 1, 0}));
    else
      XB_TRY(hy_launch(e, hy_attn_window_kernel<KT, float, 16>, dim3(T, H), dim3(32 * aw), asm_bytes, st, Q, 0, -1, (const KT*)l.k_pool,
                       (const KT*)l.k_pool, m, H, 1, W, R, W, W, far, 0, c.m_scale, 1.0f, hy->o, (long long)H * R, AttnOpt{nullptr, 0.f, 1, 0}));
  }
  return hy_launch(e, hy_head_mm_kernel<AT>, dim3((T + HY_MM_ROWS - 1) / HY_MM_ROWS, H), dim3(128), mm2, st, (const float*)hy->o,
                   (long long)H * R, (const bf16*)l.w_uv, a1, (long long)l.n_o, T, R, dv);
}

// ----------------------------------------------------------------------------- parallel blocks
// x <- embed * scale;  per layer: h = norm(x) (made by the previous row op), x += mixer(h) + ff(h).
// The mixers: latent attention (cache = latent + rotated key part, queries folded into the latent space so that a step
// never rebuilds keys or values of earlier tokens), general delta rule, lightning; feed-forwards: clamped GLU, dense or experts.
// xin: the normed stream as a Linear input [T, dim] of AT
template <typename AT>
static int hy_ff_parallel(xb_engine* e, const HyLayer& l, int T, const void* xin, cudaStream_t st, LinOut* y, LinOut* up_out = nullptr) {
  HyModel* hy = e->hy;
  const xb_hybrid_layer& c = l.d;
  const int D = hy->d.dim;
  AT* a2 = reinterpret_cast<AT*>(hy->a2);
  // Steps of so few rows that at most half of the experts can have a token: read the chosen experts' rows only (two kernels
  // in place of the wide up Linear, the activation and the wide down Linear).
  if (c.ff_kind == XB_FF_MOE && hy->use_gather && c.ff_act != XB_ACT_GELU && c.shared_ff <= 0 && l.b_up == nullptr && l.b_down == nullptr && D % 8 == 0 && c.ff % 8 == 0 &&
      2LL * T * c.top <= c.n_experts) {
    XB_TRY(hy_launch(e, hy_router_logits_kernel<AT, 1>, dim3((unsigned)(((long long)T * c.n_experts + 7) / 8)), dim3(256), 0, st,
                     reinterpret_cast<const AT*>(xin), (long long)D, (const bf16*)l.w_router, hy->m2, T, c.n_experts, D));
    const size_t rs = (size_t)4 * (2 * c.n_experts + (c.groups > 0 ? c.groups : 1)) * sizeof(float);
    XB_TRY(hy_launch(e, hy_route_kernel, dim3((T + 3) / 4), dim3(128), rs, st, (const float*)hy->m2, c.n_experts, c.top, c.groups,
                     c.keep_groups, c.route_scale, hy->gw, T, c.route_score, c.group_score, c.route_norm));
    const long long nu = (long long)T * c.top * c.ff, nd = (long long)T * D;
    XB_TRY(hy_launch(e, hy_moe_gather_up_kernel<AT>, dim3((unsigned)((nu + 7) / 8)), dim3(256), 0, st, reinterpret_cast<const AT*>(xin), (long long)D,
                     (const bf16*)l.w_up, (const float*)hy->gw, c.n_experts, c.top, c.ff, D, c.ff_limit, c.ff_act, c.route_input, a2, T));
    XB_TRY(hy_launch(e, hy_moe_gather_down_kernel<AT>, dim3((unsigned)((nd + 7) / 8)), dim3(256), 0, st, (const AT*)a2, (const bf16*)l.w_down,
                     (const float*)hy->gw, c.n_experts, c.top, c.ff, D, hy->m2, T));   // m2: the router's logits there are spent
    *y = hy_plain(hy->m2, D);
    return 0;
  }
  LinOut U;
  XB_TRY(hy_linear<AT>(e, xin, D, l.w_up, l.t_up, l.b_up, T, l.n_up, D, hy->P, hy->cap_P, st, &U));
  if (up_out != nullptr) *up_out = U;   // rows behind the experts' (a residual gate) are read by the caller
  // a bf16 matrix out of the tcgen05 Linear (prompts): the activations read and write 16 bytes per thread
  const bool vec = std::is_same<AT, bf16>::value && U.h != nullptr && U.ld % 8 == 0 && l.n_dn % 8 == 0;
  if (c.ff_kind == XB_FF_GLU_CLAMP) {
    const long long n = (long long)T * c.ff;
    if (vec && c.ff % 8 == 0)
      XB_TRY(hy_launch(e, hy_glu_clamp_vec_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), 0, st, U.h, U.ld, U.bias, c.ff, c.ff_limit,
                       reinterpret_cast<bf16*>(hy->a2), (long long)l.n_dn, T));
    else
      XB_TRY(hy_launch(e, hy_glu_clamp_kernel<AT>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, U, c.ff, c.ff_limit, a2, (long long)l.n_dn, T));
  } else {
    // router in fp32 whatever the serving type: fp32 accumulation of the products, fp32 logits
    if (T <= 64 && hy->fuse_router) {   // few rows: logits and routing of a token in one block
      const size_t rs1 = (size_t)(3 * c.n_experts + (c.groups > 0 ? c.groups : 1)) * sizeof(float);
      XB_TRY(hy_launch(e, hy_router_route_kernel<AT>, dim3(T), dim3(256), rs1, st, reinterpret_cast<const AT*>(xin), (long long)D, (const bf16*)l.w_router, D,
                       c.n_experts, c.top, c.groups, c.keep_groups, c.route_scale, hy->gw, c.route_score, c.group_score, c.route_norm));
    } else {
      if (T <= 64) {   // few rows: a warp per (token, expert)
        XB_TRY(hy_launch(e, hy_router_logits_kernel<AT, 1>, dim3((unsigned)(((long long)T * c.n_experts + 7) / 8)), dim3(256), 0, st,
                         reinterpret_cast<const AT*>(xin), (long long)D, (const bf16*)l.w_router, hy->m2, T, c.n_experts, D));
      } else {
        const int chunks = (c.n_experts + 7) / 8;
        XB_TRY(hy_launch(e, hy_router_logits_kernel<AT, 8>, dim3((unsigned)(((long long)T * chunks + 7) / 8)), dim3(256), 0, st,
                         reinterpret_cast<const AT*>(xin), (long long)D, (const bf16*)l.w_router, hy->m2, T, c.n_experts, D));
      }
      const size_t rs = (size_t)4 * (2 * c.n_experts + (c.groups > 0 ? c.groups : 1)) * sizeof(float);
      XB_TRY(hy_launch(e, hy_route_kernel, dim3((T + 3) / 4), dim3(128), rs, st, (const float*)hy->m2, c.n_experts, c.top, c.groups, c.keep_groups,
                       c.route_scale, hy->gw, T, c.route_score, c.group_score, c.route_norm));
    }
    const long long n = (long long)T * l.n_dn;
    const int sf = c.shared_ff > 0 ? c.shared_ff : 0;
    if (c.ff_act == XB_ACT_GELU) {   // experts without a gate projection
      if (vec && c.ff % 8 == 0 && sf % 8 == 0)
        XB_TRY(hy_launch(e, hy_moe_act1_vec_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), 0, st, U.h, U.ld, (const float*)hy->gw, c.n_experts,
                         c.ff, sf, reinterpret_cast<bf16*>(hy->a2), (long long)l.n_dn, T));
      else
        XB_TRY(hy_launch(e, hy_moe_act1_kernel<AT>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, U, (const float*)hy->gw, c.n_experts, c.ff, sf,
                         a2, (long long)l.n_dn, T));
    } else if (vec && c.ff % 8 == 0 && sf % 8 == 0)
      XB_TRY(hy_launch(e, hy_moe_act_vec_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), 0, st, U.h, U.ld, (const float*)hy->gw, c.n_experts,
                       c.ff, c.ff_limit, sf, c.shared_limit, c.ff_act, c.route_input, reinterpret_cast<bf16*>(hy->a2), (long long)l.n_dn, T));
    else
      XB_TRY(hy_launch(e, hy_moe_act_kernel<AT>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, U, (const float*)hy->gw, c.n_experts, c.ff,
                       c.ff_limit, sf, c.shared_limit, c.ff_act, c.route_input, a2, (long long)l.n_dn, T));
  }
  return hy_linear<AT>(e, a2, l.n_dn, l.w_down, l.t_down, l.b_down, T, D, l.n_dn, hy->m2, hy->cap_m, st, y);
}

template <typename AT>
static int hy_run_parallel_t(xb_engine* e, int T, int n_seqs, void* const* taps, cudaStream_t st, int with_head) {
  HyModel* hy = e->hy;
  const xb_hybrid_desc& d = hy->d;
  typedef typename std::conditional<std::is_same<AT, float>::value, float, bf16>::type KT;
  BatchMeta m;
  fill_batch_meta(e, m);
  m.page_table = e->d_page_table;
  m.tile_start = e->d_tile_start;
  m.tile_len = e->d_tile_len;
  m.max_pages = e->max_pages;
  m.page_tokens = e->page_tokens;
  const int D = d.dim;
  const long long SS = (long long)hy->state_floats;
  const int nwm = d.norm_scalar ? 2 : 1;
  hy->pdl_now = T <= 128;
  AT* a1 = reinterpret_cast<AT*>(hy->a1);
  AT* a2 = reinterpret_cast<AT*>(hy->a2);
  auto row_op = [&](LinOut y1, LinOut y2, const float* nw) -> int {
    RowOpArgs a;
    a.x = hy->x; a.m1 = y1; a.m2 = y2; a.m3 = hy_none(); a.s1 = 1.f; a.s2 = 1.f; a.bw = nullptr; a.bw_one = 0.f; a.nw = nw; a.hn = hy->hn;
    a.xa = nullptr; a.ha = hy->ah; a.eps = d.norm_eps; a.D = D; a.plain_add = 1; a.nw_mode = nwm; a.groups = 1; a.res_mult = 1.f; a.ext = 0;
    return hy_row_op_launch<AT>(e, T, a, st);
  };
  XB_TRY(hy_launch(e, hy_embed_kernel, dim3(T), dim3(128), 0, st, (const int*)e->in_tokens, (const bf16*)hy->embed, hy->x, D, d.vocab,
                   d.embed_scale));
  XB_TRY(row_op(hy_none(), hy_none(), hy->L[0].norm1));
  for (int li = 0; li < d.n_layers; ++li) {
    const HyLayer& l = hy->L[li];
    const xb_hybrid_layer& c = l.d;
    const float* next_norm = li + 1 < d.n_layers ? hy->L[li + 1].norm1 : hy->final_norm;
    LinOut P, y1, y2 = hy_none();
    XB_TRY(hy_linear<AT>(e, hy->ah, D, l.w_in, l.t_in, l.b_in, T, l.n_in, D, hy->P, hy->cap_P, st, &P));
    const int H = c.m_heads, n = c.m_dim;
    if (c.mixer == XB_MIX_LATENT) {
      XB_TRY(hy_latent_mixer<AT>(e, l, T, P, m, st));
    } else if (c.mixer == XB_MIX_GDELTA) {
      const int HN = H * n, rk = c.m_rank;
      LinOut Wd;
      XB_TRY(hy_launch(e, hy_act_cols_kernel<AT>, dim3(T, (rk + 255) / 256), dim3(256), 0, st, P, l.off_w1, rk, 1, a2, (long long)rk));
      XB_TRY(hy_linear<AT>(e, a2, rk, l.w_d2, l.t_d2, nullptr, T, HN, rk, hy->m2, hy->cap_m, st, &Wd));
      XB_TRY(hy_launch(e, hy_gdelta_prep_kernel, dim3(T, (H + 7) / 8), dim3(256), 0, st, P, l.off_r, l.off_k, l.off_v, l.off_a, Wd, (const float*)l.w0,
                       hy->c, (long long)6 * HN, hy->beta, hy->decay, H, n));
      RecurIn in;
      in.c = hy->c; in.ldc = 6LL * HN; in.qoff = 0; in.koff = HN; in.xoff[0] = 2LL * HN; in.xoff[1] = 3LL * HN; in.xoff[2] = 4LL * HN;
      in.voff = 5LL * HN; in.q_heads = H; in.beta = hy->beta; in.decay = hy->decay; in.qk = nullptr; in.hdecay = nullptr;
      XB_TRY(hy_recur<HY_REC_GDELTA>(e, in, hy->state + l.st_rec, SS, hy->o, (long long)l.n_o, m, n_seqs, H, n, n, st));
      XB_TRY(hy_launch(e, hy_head_norm_kernel<AT>, dim3(T, (H + 7) / 8), dim3(256), 0, st, (const float*)hy->o, (long long)l.n_o,
                       (const float*)l.head_norm, P, l.off_g, d.norm_eps, 1.0f, a1, (long long)l.n_o, H, n, n, 1));
    } else {
      const int dv = c.m_vdim;
      const int nc = 2 * H * n + H * dv;
      XB_TRY(hy_launch(e, hy_act_cols_kernel<float>, dim3(T, (nc + 255) / 256), dim3(256), 0, st, P, l.off_q, nc, 0, hy->c, (long long)nc));
      RecurIn in;
      in.c = hy->c; in.ldc = nc; in.qoff = 0; in.koff = (long long)H * n; in.voff = 2LL * H * n; in.q_heads = H;
      in.xoff[0] = in.xoff[1] = in.xoff[2] = 0;
      in.beta = in.decay = in.qk = nullptr; in.hdecay = l.hdecay;
      XB_TRY(hy_recur<HY_REC_LIGHTNING>(e, in, hy->state + l.st_rec, SS, hy->o, (long long)l.n_o, m, n_seqs, H, n, dv, st));
      XB_TRY(hy_launch(e, hy_all_heads_norm_kernel<AT>, dim3(T), dim3(256), 0, st, (const float*)hy->o, (long long)l.n_o,
                       (const float*)l.head_norm, P, l.off_g, d.norm_eps, a1, (long long)l.n_o, H * dv));
    }
    XB_TRY(hy_linear<AT>(e, a1, l.n_o, l.w_o, l.t_o, nullptr, T, D, l.n_o, hy->m1, hy->cap_m, st, &y1));
    if (c.ff > 0) XB_TRY(hy_ff_parallel<AT>(e, l, T, hy->ah, st, &y2));
    XB_TRY(row_op(y1, y2, next_norm));
    if (taps != nullptr && taps[li] != nullptr)
      XB_CUDA(cudaMemcpyAsync(taps[li], hy->x, (size_t)T * D * sizeof(float), cudaMemcpyDeviceToDevice, st));
  }
  if (with_head) {
    const int nr = e->sel_rows != nullptr ? e->sel_n : n_seqs;
    if (nr > 0) {
      const int* idx = e->sel_rows != nullptr ? hy->d_rows : m.seq_last;
      LinOut y;
      XB_TRY(hy_launch(e, hy_gather_rows_kernel<AT>, dim3(nr), dim3(256), 0, st, (const float*)hy->hn, idx, reinterpret_cast<AT*>(hy->head_in), D));
      XB_TRY(hy_linear<AT>(e, hy->head_in, D, hy->head, hy->t_head, nullptr, nr, d.vocab, D, hy->head_raw, hy->cap_head, st, &y));
      const long long tot = (long long)nr * d.vocab;
      XB_TRY(hy_launch(e, hy_logits_kernel, dim3((unsigned)((tot + 255) / 256)), dim3(256), 0, st, y, d.logit_softcap, e->logits, nr, d.vocab));
    }
  }
  return 0;
}

// Rotary-position softmax attention of one layer: P = [q | k | v | head gates] of the step's rows -> a1 = what the output
// projection reads.  Rotation, value blending and the cache append are one kernel; the attention runs a block per
// (token, head) over the pages; mixed heads / head gates follow in a kernel of their own.
// mixed heads / head gates behind the tensor-core attention kernels, whose output is a bf16 matrix in hy->o
template <typename AT>
static int hy_heads_mix_bf16(xb_engine* e, const HyLayer& l, int T, const LinOut& P, cudaStream_t st) {
  HyModel* hy = e->hy;
  const xb_hybrid_layer& c = l.d;
  const int H = c.s_heads, G = l.v_all ? c.s_kv_heads : 1, dv = c.s_vdim;
  const float* talk = c.s_talk ? (const float*)l.talk : (const float*)nullptr;
  AT* a1 = reinterpret_cast<AT*>(hy->a1);
  if (dv % 8 == 0)
    return hy_launch(e, hy_heads_mix_vec_kernel<AT>, dim3(T, (H * dv / 8 + 255) / 256), dim3(256), 0, st, (const bf16*)hy->o, talk, P,
                     c.s_gate ? l.off_g : -1, H, G, dv, a1, (long long)l.n_o);
  return hy_launch(e, hy_heads_mix_kernel<AT, bf16>, dim3(T, (H * dv + 255) / 256), dim3(256), 0, st, (const bf16*)hy->o, talk, P,
                   c.s_gate ? l.off_g : -1, H, G, dv, a1, (long long)l.n_o);
}

template <typename AT>
static int hy_softmax_mixer(xb_engine* e, const HyLayer& l, int T, int n_seqs, int n_tiles, const LinOut& P, const BatchMeta& m, cudaStream_t st) {
  HyModel* hy = e->hy;
  const xb_hybrid_layer& c = l.d;
  typedef typename std::conditional<std::is_same<AT, float>::value, float, bf16>::type KT;
  AT* a1 = reinterpret_cast<AT*>(hy->a1);
  const int H = c.s_heads, G = c.s_kv_heads, dk = c.s_dim, dv = c.s_vdim;
  RotArgs r;
  r.freq = l.rot_freq_d; r.dims = c.s_rot_dims; r.half = c.s_rot_pairs == XB_ROPE_HALF_SPLIT ? 1 : 0; r.mult = c.s_rot_mult;
  const int units = (H + G) * (dk - c.s_rot_dims / 2) + G * dv;
  // prompts in bf16 serving at the head sizes it takes: the tcgen05 kernel over the step's query tiles
  const bool tc = std::is_same<AT, bf16>::value && l.tc_attn && hy->use_tc_attn && n_tiles > 0;
  // steps of single tokens, same sizes: the split-key decode kernel (its splits merge inside a cluster)
  const bool dec = std::is_same<AT, bf16>::value && l.tc_attn && hy->use_tc_attn && n_tiles == 0 && T == n_seqs && e->attn_cluster != 0;
  // prompts: a block walks all units of its token (the row's position, page and angles are fetched once); few rows: a block
  // per 256 units so that the step fills more SMs
  const int rope_by = T >= 512 ? 1 : (units + 255) / 256;
  const bool rope_vec = tc && P.h != nullptr && P.bias == nullptr && P.ld % 8 == 0 && dk % 8 == 0 && dv % 8 == 0 &&
                        c.s_rot_dims % (r.half ? 16 : 8) == 0 && (G * dv) % 8 == 0;
  if (c.s_qk_norm != 0 || c.s_v_is_k != 0 || c.s_qtemp_every > 0) {   // no rotation: whole-projection norms, temperature, append
    const float* qn = c.s_qk_norm ? (const float*)l.qn : (const float*)nullptr;
    const float* kn = c.s_qk_norm ? (const float*)l.kn : (const float*)nullptr;
    float* qa = (tc || dec) ? (float*)nullptr : hy->qa;          // fp32 queries for the per-(token, head) kernel only
    bf16* qg = (tc || dec) ? hy->qg : (bf16*)nullptr;
    const size_t sm = (size_t)(H + G) * dk * sizeof(float);
    bool vec8 = false;   // a prompt whose projection came back as a bf16 matrix, bf16 pools: 16 bytes per thread
    if constexpr (std::is_same<KT, bf16>::value)
      vec8 = T > 64 && qg != nullptr && qa == nullptr && P.h != nullptr && P.ld % 8 == 0 && dk % 8 == 0 && dv % 8 == 0 && l.off_q % 8 == 0 &&
             l.off_k % 8 == 0 && l.off_v % 8 == 0;
    if (vec8) {
      if constexpr (std::is_same<KT, bf16>::value)
        XB_TRY(hy_launch(e, hy_qk_prep_vec_kernel, dim3(T), dim3(256), sm, st, P.h, P.ld, P.bias, l.off_q, l.off_k, l.off_v, H, G, dk, dv, qn, kn,
                         hy->d.norm_eps, c.s_qtemp_coef, c.s_qtemp_every, qg, (bf16*)l.k_pool, (bf16*)l.v_pool, m));
    } else if (T <= 64)
      XB_TRY(hy_launch(e, hy_qk_prep_kernel<KT, 1024>, dim3(T), dim3(1024), sm, st, P, l.off_q, l.off_k, l.off_v, H, G, dk, dv, qn, kn, hy->d.norm_eps,
                       c.s_qtemp_coef, c.s_qtemp_every, qa, qg, (KT*)l.k_pool, (KT*)l.v_pool, m));
    else
      XB_TRY(hy_launch(e, hy_qk_prep_kernel<KT, 256>, dim3(T), dim3(256), sm, st, P, l.off_q, l.off_k, l.off_v, H, G, dk, dv, qn, kn, hy->d.norm_eps,
                       c.s_qtemp_coef, c.s_qtemp_every, qa, qg, (KT*)l.k_pool, (KT*)l.v_pool, m));
  }
  else if (rope_vec)   // a prompt whose projection came back as a bf16 matrix: 16 bytes per thread
    XB_TRY(hy_launch(e, hy_rope_append_vec_kernel, dim3(T), dim3(256), 0, st, P.h, P.ld, l.off_q, l.off_k, l.off_v, H, G, dk, dv, r, hy->qg,
                     (bf16*)l.k_pool, (bf16*)l.v_pool, l.v_all ? 1 : 0, (const float*)l.vmix, hy->vfirst, l.vmode, m));
  else
  XB_TRY(hy_launch(e, hy_rope_append_kernel<KT>, dim3(T, rope_by), dim3(256), 0, st, P, l.off_q, l.off_k, l.off_v, H, G, dk, dv, r,
                   hy->qa, (tc || dec) ? hy->qg : (bf16*)nullptr, (KT*)l.k_pool, (KT*)l.v_pool, l.v_all ? 1 : 0, (const float*)l.vmix, hy->vfirst,
                   l.vmode, m));
  const int dvo = l.v_all ? G * dv : dv;
  const int vch = dvo > 512 ? 512 : 0;   // wider value rows: blocks along z take 512 channels each
  const AttnOpt opt{c.s_sink ? l.sink : nullptr, c.s_softcap, l.v_all ? 1 : G, vch, c.s_dist_bias ? l.r1 : nullptr, c.s_dist_bias ? l.r2 : nullptr};
  const bool post = c.s_talk != 0 || c.s_gate != 0;
  if (dec) {
    // mixed heads multiply the blocks by the key heads: fewer splits keep the grid near one wave
    int ns = l.v_all ? hy->dec_splits / G : hy->dec_splits;
    ns = ns < 1 ? 1 : ns;
    const AttDecOpt dopt{c.s_sink ? l.sink : nullptr, c.s_softcap, l.v_all ? 1 : 0, (long long)dvo, hy->p_split, opt.r1, opt.r2};
    bf16* dst = post ? reinterpret_cast<bf16*>(hy->o) : reinterpret_cast<bf16*>(hy->a1);
    if (dk == 128) XB_TRY(hy_attn_dec<128>(e, l, m, T, hy->qg, dst, H, G, c.s_scale, ns, dopt, st));
    else XB_TRY(hy_attn_dec<64>(e, l, m, T, hy->qg, dst, H, G, c.s_scale, ns, dopt, st));
    if (post) XB_TRY(hy_heads_mix_bf16<AT>(e, l, T, P, st));
    return 0;
  }
  if (tc) {
    HyAttnIn in;
    in.tile_start = m.tile_start; in.tile_len = m.tile_len; in.n_tiles = n_tiles; in.q = hy->qg;
    in.io = AttIo{(long long)H * dk, nullptr, nullptr, 0, c.s_sink ? l.sink : nullptr, c.s_softcap, l.v_all ? 1 : 0, (long long)dvo, hy->p_split, opt.r1, opt.r2};
    bf16* dst = post ? reinterpret_cast<bf16*>(hy->o) : reinterpret_cast<bf16*>(hy->a1);
    if (dk == 128) XB_TRY(hy_attn_tc_any<128>(e, l, m, in, dst, H, G, c.s_scale, l.v_all ? G : 1, st));
    else XB_TRY(hy_attn_tc_any<64>(e, l, m, in, dst, H, G, c.s_scale, l.v_all ? G : 1, st));
    if (post) XB_TRY(hy_heads_mix_bf16<AT>(e, l, T, P, st));
    return 0;
  }
  const int aw = 16, far = 1 << 30;   // causal over the whole sequence: the block's warps share out all earlier keys
  const size_t asm_bytes = (size_t)(((dk + 3) & ~3) + aw * (2 + (vch ? vch : dvo))) * sizeof(float);
  const LinOut Q = hy_plain(hy->qa, (long long)H * dk);
  const KT* kp = (const KT*)l.k_pool;
  const KT* vp = (const KT*)l.v_pool;
  const dim3 grid(T, H, vch ? (dvo + vch - 1) / vch : 1), block(32 * aw);
  if (post) {
    if (dvo <= 256)
      XB_TRY(hy_launch(e, hy_attn_window_kernel<KT, float, 8>, grid, block, asm_bytes, st, Q, 0, -1, kp, vp, m, H, G, dk, dvo, dk, dvo, far, 0,
                       c.s_scale, 1.0f, hy->o, (long long)H * dvo, opt));
    else
      XB_TRY(hy_launch(e, hy_attn_window_kernel<KT, float, 16>, grid, block, asm_bytes, st, Q, 0, -1, kp, vp, m, H, G, dk, dvo, dk, dvo, far, 0,
                       c.s_scale, 1.0f, hy->o, (long long)H * dvo, opt));
    XB_TRY(hy_launch(e, hy_heads_mix_kernel<AT, float>, dim3(T, (H * dv + 255) / 256), dim3(256), 0, st, (const float*)hy->o,
                     c.s_talk ? (const float*)l.talk : (const float*)nullptr, P, c.s_gate ? l.off_g : -1, H, l.v_all ? G : 1, dv, a1, (long long)l.n_o));
  } else {
    if (dvo <= 256)
      XB_TRY(hy_launch(e, hy_attn_window_kernel<KT, AT, 8>, grid, block, asm_bytes, st, Q, 0, -1, kp, vp, m, H, G, dk, dvo, dk, dvo, far, 0,
                       c.s_scale, 1.0f, a1, (long long)l.n_o, opt));
    else
      XB_TRY(hy_launch(e, hy_attn_window_kernel<KT, AT, 16>, grid, block, asm_bytes, st, Q, 0, -1, kp, vp, m, H, G, dk, dvo, dk, dvo, far, 0,
                       c.s_scale, 1.0f, a1, (long long)l.n_o, opt));
  }
  return 0;
}

// ----------------------------------------------------------------------------- branch-norm blocks
// x <- embedding rows (token + token pair + position);  per layer  x += n1 unit(g1 * mixer(x)),  x += n2 unit(g2 * ff(x)),
// g = sigmoid(W x + b) with the gate's rows riding in the sublayer's own input projection.  What a sublayer reads is the
// stream itself (as a Linear input: xa, written by the kernel that last changed x); only the model's last norm exists as a row.
template <typename AT>
static int hy_run_branchnorm_t(xb_engine* e, int T, int n_seqs, int n_tiles, void* const* taps, cudaStream_t st, int with_head) {
  HyModel* hy = e->hy;
  const xb_hybrid_desc& d = hy->d;
  BatchMeta m;
  fill_batch_meta(e, m);
  m.page_table = e->d_page_table;
  m.tile_start = e->d_tile_start;
  m.tile_len = e->d_tile_len;
  m.max_pages = e->max_pages;
  m.page_tokens = e->page_tokens;
  const int D = d.dim;
  const long long SS = (long long)hy->state_floats;
  hy->pdl_now = T <= 128;
  AT* a1 = reinterpret_cast<AT*>(hy->a1);
  const bool few = T <= 64 && D >= 1024;
  auto row_op = [&](const LinOut& y, const LinOut& P, int off_gate, const float* bw, const float* nw) -> int {
    RowOpArgs a;
    a.x = hy->x; a.m1 = y; a.m2 = hy_none(); a.m3 = hy_none(); a.s1 = 1.f; a.s2 = 0.f; a.bw = bw; a.bw_one = 0.f; a.nw = nw; a.hn = hy->hn;
    a.xa = a1; a.ha = nullptr; a.eps = d.norm_eps; a.D = D; a.plain_add = 0; a.nw_mode = d.norm_scalar ? 2 : 1; a.groups = 1; a.res_mult = 1.f; a.ext = 0;
    a.gate = off_gate >= 0 ? P : hy_none(); a.gate_off = off_gate >= 0 ? off_gate : 0; a.bw_mode = d.norm_scalar ? 2 : 1;
    // prompts whose branch and gate came back as bf16 matrices: eight channels per thread
    const bool gate_ok = off_gate < 0 || (P.h != nullptr && P.ld % 8 == 0 && off_gate % 8 == 0);
    if (!few && y.h != nullptr && y.bias == nullptr && y.ld % 8 == 0 && gate_ok && D % 8 == 0)
      return hy_launch(e, hy_row_op_gated_vec_kernel<AT>, dim3(T), dim3(256), (size_t)D * sizeof(float), st, a);
    if (few) return hy_launch(e, hy_row_op_gated_kernel<AT, 1024>, dim3(T), dim3(1024), (size_t)D * sizeof(float), st, a);
    return hy_launch(e, hy_row_op_gated_kernel<AT, 256>, dim3(T), dim3(256), (size_t)D * sizeof(float), st, a);
  };
  const bool single = T == n_seqs;   // a step of single tokens: every row is its sequence's last
  float* prev = hy->state + hy->st_prev;
  XB_TRY(hy_launch(e, hy_embed_sum_kernel<AT>, dim3(T), dim3(128), 0, st, (const int*)e->in_tokens, (const bf16*)hy->embed, (const bf16*)hy->bigram,
                   (const bf16*)hy->pos_tab, hy->x, a1, D, d.vocab, d.embed_scale, d.bigram_buckets, d.bigram_mul_prev, d.bigram_mul_cur, d.pos_rows,
                   prev, SS, single ? 1 : 0, m));
  if (hy->bigram != nullptr && !single)
    XB_TRY(hy_launch(e, hy_prev_token_kernel, dim3((n_seqs + 127) / 128), dim3(128), 0, st, (const int*)e->in_tokens, prev, SS, d.vocab, n_seqs, m));
  for (int li = 0; li < d.n_layers; ++li) {
    const HyLayer& l = hy->L[li];
    const xb_hybrid_layer& c = l.d;
    const bool has_ff = c.ff > 0;
    const bool last = li + 1 == d.n_layers;
    LinOut P, y1;
    XB_TRY(hy_linear<AT>(e, a1, D, l.w_in, l.t_in, l.b_in, T, l.n_in, D, hy->P, hy->cap_P, st, &P));
    if (c.mixer == XB_MIX_LATENT) XB_TRY(hy_latent_mixer<AT>(e, l, T, P, m, st));
    else XB_TRY(hy_softmax_mixer<AT>(e, l, T, n_seqs, n_tiles, P, m, st));
    XB_TRY(hy_linear<AT>(e, a1, l.n_o, l.w_o, l.t_o, nullptr, T, D, l.n_o, hy->m1, hy->cap_m, st, &y1));
    XB_TRY(row_op(y1, P, l.off_rg, l.norm1, (last && !has_ff) ? hy->final_norm : nullptr));
    if (has_ff) {
      LinOut dn, U;
      XB_TRY(hy_ff_parallel<AT>(e, l, T, a1, st, &dn, &U));
      XB_TRY(row_op(dn, U, l.off_rg2, l.norm2, last ? hy->final_norm : nullptr));
    }
    if (taps != nullptr && taps[li] != nullptr)
      XB_CUDA(cudaMemcpyAsync(taps[li], hy->x, (size_t)T * D * sizeof(float), cudaMemcpyDeviceToDevice, st));
  }
  if (with_head) {
    const int n = e->sel_rows != nullptr ? e->sel_n : n_seqs;
    if (n > 0) {
      const int* idx = e->sel_rows != nullptr ? hy->d_rows : m.seq_last;
      LinOut y;
      XB_TRY(hy_launch(e, hy_gather_rows_kernel<AT>, dim3(n), dim3(256), 0, st, (const float*)hy->hn, idx, reinterpret_cast<AT*>(hy->head_in), D));
      XB_TRY(hy_linear<AT>(e, hy->head_in, D, hy->head, hy->t_head, nullptr, n, d.vocab, D, hy->head_raw, hy->cap_head, st, &y));
      const long long tot = (long long)n * d.vocab;
      XB_TRY(hy_launch(e, hy_logits_kernel, dim3((unsigned)((tot + 255) / 256)), dim3(256), 0, st, y, d.logit_softcap, e->logits, n, d.vocab));
    }
  }
  return 0;
}

template <typename AT>
static int hy_run_body_t(xb_engine* e, int T, int n_seqs, int n_tiles, void* const* taps, cudaStream_t st, int with_head) {
  HyModel* hy = e->hy;
  const xb_hybrid_desc& d = hy->d;
  if (d.block == XB_BLOCK_PARALLEL) return hy_run_parallel_t<AT>(e, T, n_seqs, taps, st, with_head);
  if (d.block == XB_BLOCK_BRANCHNORM) return hy_run_branchnorm_t<AT>(e, T, n_seqs, n_tiles, taps, st, with_head);
  typedef typename std::conditional<std::is_same<AT, float>::value, float, bf16>::type KT;
  BatchMeta m;
  fill_batch_meta(e, m);
  m.page_table = e->d_page_table;
  m.tile_start = e->d_tile_start;
  m.tile_len = e->d_tile_len;
  m.max_pages = e->max_pages;
  m.page_tokens = e->page_tokens;
  const int D = d.dim;
  const long long SS = (long long)hy->state_floats;
  hy->pdl_now = T <= 128;
  const bool no_span = T == n_seqs;    // a step of single tokens: no sequence spans two filter tiles
  // few rows: the per-layer token input (two small Linears, gate, norm, residual) in one kernel, a block per row
  const bool side_fused = T <= 64 && (size_t)(2 * D + d.side_dim + 8) * sizeof(float) <= 48 * 1024;
  AT* a1 = reinterpret_cast<AT*>(hy->a1);
  AT* a2 = reinterpret_cast<AT*>(hy->a2);
  XB_TRY(hy_launch(e, hy_embed_kernel, dim3(T), dim3(128), 0, st, (const int*)e->in_tokens, (const bf16*)hy->embed, hy->x, D, d.vocab,
                   d.embed_scale));
  XB_TRY(hy_row_op<AT>(e, T, hy_none(), 0.f, hy_none(), 0.f, nullptr, 0.f, hy->L[0].norm1, nullptr, st));
  for (int li = 0; li < d.n_layers; ++li) {
    const HyLayer& l = hy->L[li];
    const xb_hybrid_layer& c = l.d;
    const float* next_norm = li + 1 < d.n_layers ? hy->L[li + 1].norm1 : hy->final_norm;
    const bool has_ff = c.ff > 0, has_side = d.side_dim > 0;
    LinOut P, y1, y2 = hy_none();
    float s1 = 1.f, s2 = 0.f;
    XB_TRY(hy_sublayer_input<AT>(e, T, n_seqs, no_span, l.canon1, l.st_canon1, m, st));
    XB_TRY(hy_linear<AT>(e, a1, D, l.w_in, l.t_in, l.b_in, T, l.n_in, D, hy->P, hy->cap_P, st, &P));
    if (c.mixer == XB_MIX_DELTA) {
      const int H = c.d_heads, G = c.d_kv_heads, dk = c.d_dim, dv = c.d_vdim, tp = c.d_taps;
      float* tail = hy->state + l.st_conv;
      XB_TRY(hy_filter<float>(e, T, n_seqs, no_span, P, 0, l.c_conv, tp, l.conv_w, tail, m, 0, 1, hy->c, (long long)l.c_conv, st));
      XB_TRY(hy_launch(e, hy_delta_prep_kernel, dim3(T), dim3(256), 0, st, hy->c, (long long)l.c_conv, P, l.off_b, l.off_a,
                       (const float*)l.A_log, (const float*)l.dt_bias, hy->beta, hy->decay, hy->qk, H, G, dk));
      {
        RecurIn in;
        in.c = hy->c; in.ldc = l.c_conv; in.qoff = 0; in.koff = (long long)G * dk; in.voff = 2LL * G * dk; in.q_heads = G;
        in.beta = hy->beta; in.decay = hy->decay; in.qk = hy->qk; in.hdecay = nullptr;
        in.xoff[0] = in.xoff[1] = in.xoff[2] = 0;
        XB_TRY(hy_recur<HY_REC_DELTA>(e, in, hy->state + l.st_rec, SS, hy->o, (long long)l.n_o, m, n_seqs, H, dk, dv, st));
      }
      XB_TRY(hy_launch(e, hy_head_norm_kernel<AT>, dim3(T, (H + 7) / 8), dim3(256), 0, st, (const float*)hy->o, (long long)l.n_o,
                       (const float*)l.head_norm, P, l.off_g, d.norm_eps, 1.0f, a1, (long long)l.n_o, H, dv, 0, 0));
      XB_TRY(hy_linear<AT>(e, a1, l.n_o, l.w_o, l.t_o, nullptr, T, D, l.n_o, hy->m1, hy->cap_m, st, &y1));
    } else if (c.mixer == XB_MIX_SOFTMAX) {
      XB_TRY(hy_softmax_mixer<AT>(e, l, T, n_seqs, n_tiles, P, m, st));
      XB_TRY(hy_linear<AT>(e, a1, l.n_o, l.w_o, l.t_o, nullptr, T, D, l.n_o, hy->m1, hy->cap_m, st, &y1));
    } else {
      const int H = c.a_heads, G = c.a_kv_heads, dk = c.a_dim, dv = c.a_vdim;
      const int Hr = c.r_heads, rk = c.r_dim, rv = c.r_vdim;
      XB_TRY(hy_launch(e, hy_kv_append_kernel<KT>, dim3(T, (G * (dk + dv) + 255) / 256), dim3(256), 0, st, P, l.off_k, l.off_v, (KT*)l.k_pool, (KT*)l.v_pool, m, G, dk, dv));
      // bf16 serving at the head sizes it takes: the tcgen05 kernel, over the step's query tiles (a step of single tokens:
      // one tile per sequence).  It reads q and the gate as bf16 rows: straight from the projection when that came back
      // as a bf16 matrix (16-byte loads need aligned pitches), else from a packed copy of the split-K planes.
      const bool single = T == n_seqs;
      const bool tc = std::is_same<AT, bf16>::value && l.tc_attn && hy->use_tc_attn && (n_tiles > 0 || single);
      if (tc) {
        HyAttnIn in;
        in.tile_start = n_tiles > 0 ? m.tile_start : m.tok_seq;   // single tokens: row i is sequence i
        in.tile_len = n_tiles > 0 ? m.tile_len : hy->d_ones;
        in.n_tiles = n_tiles > 0 ? n_tiles : n_seqs;
        if (P.h != nullptr && P.ld % 8 == 0 && l.off_g % 8 == 0) {
          in.q = P.h + l.off_q;
          in.io = AttIo{P.ld, P.bias != nullptr ? P.bias + l.off_q : nullptr, P.h + l.off_g, P.ld};
        } else {
          const int nq = H * dk, ng = H * dv;
          XB_TRY(hy_launch(e, hy_qg_pack_kernel, dim3(T, (nq + ng + 255) / 256), dim3(256), 0, st, P, l.off_q, nq, l.off_g, ng, hy->qg));
          in.q = hy->qg;
          in.io = AttIo{(long long)(nq + ng), nullptr, hy->qg + nq, (long long)(nq + ng)};
        }
        if (dk == 128) XB_TRY(hy_attn_tc<128>(e, l, m, in, reinterpret_cast<bf16*>(hy->a1), st));
        else XB_TRY(hy_attn_tc<64>(e, l, m, in, reinterpret_cast<bf16*>(hy->a1), st));
      } else {
        // warps per (token, head): one per 64 visible keys, at most 16
        int aw = (c.a_window + c.a_keep_first + 63) / 64;
        aw = aw < 1 ? 1 : (aw > 16 ? 16 : aw);
        const size_t asm_bytes = (size_t)(((dk + 3) & ~3) + aw * (2 + dv)) * sizeof(float);
        XB_TRY(hy_launch(e, hy_attn_window_kernel<KT, AT, 8>, dim3(T, H), dim3(32 * aw), asm_bytes, st, P, l.off_q, l.off_g,
                         (const KT*)l.k_pool, (const KT*)l.v_pool, m, H, G, dk, dv, dk, dv, c.a_window, c.a_keep_first, c.a_scale, 1.0f, a1,
                         (long long)l.n_o, AttnOpt{nullptr, 0.f, G, 0}));
      }
      const long long ldc = 2LL * Hr * rk + (long long)Hr * rv;
      XB_TRY(hy_launch(e, hy_hgrn_prep_kernel, dim3(T, (2 * Hr * rk + Hr * rv + 255) / 256), dim3(256), 0, st, P, l.off_rq, l.off_rf, l.off_rv, (const float*)l.lower, hy->c,
                       ldc, Hr * rk, Hr * rv));
      {
        RecurIn in;
        in.c = hy->c; in.ldc = ldc; in.qoff = 0; in.koff = (long long)Hr * rk; in.voff = 2LL * Hr * rk; in.q_heads = Hr;
        in.beta = in.decay = in.qk = in.hdecay = nullptr;
        in.xoff[0] = in.xoff[1] = in.xoff[2] = 0;
        XB_TRY(hy_recur<HY_REC_HGRN>(e, in, hy->state + l.st_rec, SS, hy->o, (long long)l.n_o2, m, n_seqs, Hr, rk, rv, st));
      }
      XB_TRY(hy_launch(e, hy_head_norm_kernel<AT>, dim3(T, (Hr + 7) / 8), dim3(256), 0, st, (const float*)hy->o, (long long)l.n_o2,
                       (const float*)l.head_norm, P, -1, d.norm_eps, 1.0f, a2, (long long)l.n_o2, Hr, rv, 0, 0));
      XB_TRY(hy_linear<AT>(e, a1, l.n_o, l.w_o, l.t_o, nullptr, T, D, l.n_o, hy->m1, hy->cap_m, st, &y1));
      XB_TRY(hy_linear<AT>(e, a2, l.n_o2, l.w_o2, l.t_o2, nullptr, T, D, l.n_o2, hy->m2, hy->cap_m, st, &y2));
      s1 = c.left_scale;
      s2 = c.right_scale;
    }
    // x += norm1b(mixer); then whatever reads x next
    const bool ff_direct = has_ff && d.ff_unfiltered != 0;   // the feed-forward reads its norm without a filter
    XB_TRY(hy_row_op<AT>(e, T, y1, s1, y2, s2, l.norm1b, 1.f, has_ff ? l.norm2 : (has_side ? nullptr : next_norm),
                         (!has_ff && has_side && !side_fused) ? (void*)a1 : nullptr, st, ff_direct ? (void*)a1 : nullptr));
    if (has_ff && c.ff_kind == XB_FF_MOE) {
      LinOut dn;
      if (!ff_direct) XB_TRY(hy_sublayer_input<AT>(e, T, n_seqs, no_span, l.canon2, l.st_canon2, m, st));
      XB_TRY(hy_ff_parallel<AT>(e, l, T, a1, st, &dn));
      XB_TRY(hy_row_op<AT>(e, T, dn, 1.f, hy_none(), 0.f, l.norm2b, 1.f, has_side ? nullptr : next_norm, (has_side && !side_fused) ? (void*)a1 : nullptr, st));
    } else if (has_ff) {
      LinOut u, dn;
      if (!ff_direct) XB_TRY(hy_sublayer_input<AT>(e, T, n_seqs, no_span, l.canon2, l.st_canon2, m, st));
      XB_TRY(hy_linear<AT>(e, a1, D, l.w_up, l.t_up, nullptr, T, c.ff, D, hy->P, hy->cap_P, st, &u));
      const long long n = (long long)T * c.ff;
      if (std::is_same<AT, bf16>::value && u.h != nullptr && u.bias == nullptr && c.ff % 8 == 0 && u.ld % 8 == 0)
        XB_TRY(hy_launch(e, hy_relu2_vec_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), 0, st, u.h, u.ld, reinterpret_cast<bf16*>(hy->a1),
                         (long long)c.ff, T, c.ff));
      else
        XB_TRY(hy_launch(e, hy_relu2_kernel<AT>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, u, a1, (long long)c.ff, T, c.ff));
      XB_TRY(hy_linear<AT>(e, a1, c.ff, l.w_down, l.t_down, nullptr, T, D, c.ff, hy->m1, hy->cap_m, st, &dn));
      XB_TRY(hy_row_op<AT>(e, T, dn, 1.f, hy_none(), 0.f, l.norm2b, 1.f, has_side ? nullptr : next_norm, (has_side && !side_fused) ? (void*)a1 : nullptr, st));
    }
    if (has_side && side_fused) {
      XB_TRY(hy_launch(e, hy_side_fused_kernel<AT>, dim3(T), dim3(1024), (size_t)(2 * D + d.side_dim + 8) * sizeof(float), st, hy->x,
                       (const int*)e->in_tokens, (const bf16*)hy->side_embed, (long long)d.side_dim * d.n_layers, li * d.side_dim, d.vocab,
                       (const bf16*)l.w_sgate, (const bf16*)l.w_sproj, (const float*)l.side_norm, next_norm, hy->hn, d.norm_eps, D, d.side_dim));
    } else if (has_side) {
      LinOut gt, yy;
      const int sd = d.side_dim;
      XB_TRY(hy_linear<AT>(e, a1, D, l.w_sgate, l.t_sgate, nullptr, T, sd, D, hy->P, hy->cap_P, st, &gt));
      const long long n = (long long)T * sd;
      XB_TRY(hy_launch(e, hy_side_gate_kernel<AT>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, gt, (const int*)e->in_tokens,
                       (const bf16*)hy->side_embed, (long long)sd * d.n_layers, li * sd, d.vocab, a2, (long long)sd, T, sd));
      XB_TRY(hy_linear<AT>(e, a2, sd, l.w_sproj, l.t_sproj, nullptr, T, D, sd, hy->m1, hy->cap_m, st, &yy));
      XB_TRY(hy_row_op<AT>(e, T, yy, 1.f, hy_none(), 0.f, l.side_norm, 0.f, next_norm, nullptr, st));
    }
    if (taps != nullptr && taps[li] != nullptr)
      XB_CUDA(cudaMemcpyAsync(taps[li], hy->x, (size_t)T * D * sizeof(float), cudaMemcpyDeviceToDevice, st));
  }
  if (with_head) {
    const int n = e->sel_rows != nullptr ? e->sel_n : n_seqs;
    if (n > 0) {
      const int* idx = e->sel_rows != nullptr ? hy->d_rows : m.seq_last;
      LinOut y;
      XB_TRY(hy_launch(e, hy_gather_rows_kernel<AT>, dim3(n), dim3(256), 0, st, (const float*)hy->hn, idx, reinterpret_cast<AT*>(hy->head_in), D));
      XB_TRY(hy_linear<AT>(e, hy->head_in, D, hy->head, hy->t_head, nullptr, n, d.vocab, D, hy->head_raw, hy->cap_head, st, &y));
      const long long tot = (long long)n * d.vocab;
      XB_TRY(hy_launch(e, hy_logits_kernel, dim3((unsigned)((tot + 255) / 256)), dim3(256), 0, st, y, d.logit_softcap, e->logits, n, d.vocab));
    }
  }
  return 0;
}

static int hy_run_body(xb_engine* e, int T, int n_seqs, int n_splits, int n_tiles, void* const* taps, cudaStream_t st, int with_head) {
  e->hy->dec_splits = n_splits > 0 ? n_splits : 1;
  if (e->hy->d.compute_fp32) return hy_run_body_t<float>(e, T, n_seqs, n_tiles, taps, st, with_head);
  return hy_run_body_t<bf16>(e, T, n_seqs, n_tiles, taps, st, with_head);
}

// Key splits of a step of single tokens for the attention layers that decode through the split-key tensor-core kernel: one
// wave of about two blocks per SM over (token, key head, split), at most one cluster of splits; 1 when no layer uses it.
static int hy_kv_splits(xb_engine* e, int T, int max_ctx) {
  HyModel* hy = e->hy;
  int kv = 0;
  for (const HyLayer& l : hy->L)
    if (l.d.mixer == XB_MIX_SOFTMAX && l.tc_attn && l.d.s_kv_heads > kv) kv = l.d.s_kv_heads;
  if (kv == 0 || !e->attn_cluster || !hy->use_tc_attn) return 1;
  const int tiles = (max_ctx + XB_ATT_TILE - 1) / XB_ATT_TILE;
  int n = (2 * e->num_sms) / (T * kv);
  n = n > 8 ? 8 : n;
  n = n > tiles ? tiles : n;
  return n < 1 ? 1 : n;
}
