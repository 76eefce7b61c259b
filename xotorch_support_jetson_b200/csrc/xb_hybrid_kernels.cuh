// Kernels of the hybrid layer kinds (xb_hybrid_layer in xb200.h): gated delta rule, HGRN2, windowed softmax attention
// with kept first tokens and an output gate, causal per-channel filters with a carried tail, fp32 residual + RMS norms,
// squared-ReLU feed-forward, per-layer token side input, soft-capped logits.
//
// Precision: the residual stream, norms, attention scores and weights, gates, decays, unit norms and the recurrent
// state are fp32 everywhere.  AT is the type a Linear READS: bf16 (serving) or float (the all-fp32 mode, no TF32:
// plain FMA).  Every Linear's output is consumed through LinOut, which hides whether it is one fp32 matrix, fp32
// split-K planes of the tcgen05 kernel, or a bf16 matrix.
//
// Per-sequence state lives in slots: a sequence that starts at position 0 finds zero state whatever the slot held
// before (kernels test the position instead of clearing memory).
#pragma once
#include "xb_common.cuh"
#include "xb_kernels.cuh"
#include "xb_latent_attn.cuh"
#include <math.h>

// Every kernel of the forward opens with griddepcontrol.launch_dependents / griddepcontrol.wait: launched with the
// programmatic-serialization attribute, the next kernel's launch overlaps this one's execution and it touches upstream
// data only after the wait (the whole chain of earlier kernels has then completed).
#define HY_MAX_TAPS 16   // causal filters keep taps - 1 inputs per sequence
#define HY_MAX_KDIM 256  // recurrent state: four lanes own one value column, up to 64 rows each
// what one step does to a state column S_j (see hy_recur_kernel)
#define HY_REC_HGRN 0
#define HY_REC_DELTA 1
#define HY_REC_GDELTA 2
#define HY_REC_LIGHTNING 3

struct LinOut {
  const float* f;      // fp32 [planes][T][ld] (planes summed per column, see SplitInfo), or nullptr
  const bf16* h;       // bf16 [T][ld], or nullptr
  SplitInfo si;        // si.splits == 0: one plane
  long long plane;     // floats between planes
  long long ld;
  const float* bias;   // added on read (outputs of the tcgen05 Linear; the plain kernels add it themselves), or nullptr
};

__device__ __forceinline__ float lin_at(const LinOut& o, long long row, int col) {
  const float b = o.bias != nullptr ? o.bias[col] : 0.f;
  if (o.h != nullptr) return bf2f(o.h[row * o.ld + col]) + b;
  const float* p = o.f + row * o.ld + col;
  if (o.si.splits == 0) return *p + b;
  const int n = xb_n_segments(o.si, col);
  float s = 0.f;
  int i = 0;
  for (; i + 3 < n; i += 4) {   // four planes in flight
    const float v0 = p[i * o.plane], v1 = p[(i + 1) * o.plane], v2 = p[(i + 2) * o.plane], v3 = p[(i + 3) * o.plane];
    s += (v0 + v1) + (v2 + v3);
  }
  for (; i < n; ++i) s += p[i * o.plane];
  return s + b;
}

template <typename AT> __device__ __forceinline__ void act_store(AT* p, float v);
template <> __device__ __forceinline__ void act_store<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void act_store<bf16>(bf16* p, float v) { *p = f2bf(v); }
template <typename AT> __device__ __forceinline__ float2 act_load2(const AT* p);   // two neighbours; p 2-element aligned
template <> __device__ __forceinline__ float2 act_load2<float>(const float* p) { return *reinterpret_cast<const float2*>(p); }
template <> __device__ __forceinline__ float2 act_load2<bf16>(const bf16* p) { return bf2_to_f2(*reinterpret_cast<const uint32_t*>(p)); }
template <typename AT> __device__ __forceinline__ float act_load(const AT* p);
template <> __device__ __forceinline__ float act_load<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float act_load<bf16>(const bf16* p) { return bf2f(*p); }

__device__ __forceinline__ float hy_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float hy_silu(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float hy_softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float hy_gelu_tanh(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// first row, length, first position and slot of the sequence with index s
struct SeqSpan { int start, len, pos0, slot; };
__device__ __forceinline__ SeqSpan seq_span(const BatchMeta& m, int s) {
  SeqSpan r;
  r.start = s > 0 ? m.seq_last[s - 1] + 1 : 0;
  r.len = m.seq_last[s] - r.start + 1;
  r.pos0 = m.tok_pos[r.start];
  r.slot = m.seq_slot[s];
  return r;
}

// ----------------------------------------------------------------------------- embedding
__global__ void hy_embed_kernel(const int* __restrict__ tokens, const bf16* __restrict__ emb, float* __restrict__ x, int D, int V, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int tok = tokens[t];
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
  for (int i = threadIdx.x; i < D; i += blockDim.x) x[(long long)t * D + i] = bf2f(emb[(long long)tok * D + i]) * scale;
}

// Embedding as a sum of three rows: the token's, a hashed row of the (previous token, token) pair and a learned position row.
//   x[t] = emb[tok] * scale + bigram[(prev * mul_prev + tok * mul_cur) mod buckets] + pos_tab[position]
// A sequence's first token (position 0) takes row `buckets` of the pair table.  The previous token of a row that opens a
// step's portion comes from the slot's state (prev_state[slot * SS], the token's bits in a float), written by the step that
// ran the token before it.  write_prev: a step of single tokens, where the row is also its sequence's last, stores its own
// token there; other steps launch hy_prev_token_kernel behind this kernel (a block of another row may still read the word).
// xa: the row as a Linear input.  bigram / pos_tab may be nullptr (that term is absent).
template <typename AT>
__global__ void hy_embed_sum_kernel(const int* __restrict__ tokens, const bf16* __restrict__ emb, const bf16* __restrict__ bigram,
                                    const bf16* __restrict__ pos_tab, float* __restrict__ x, AT* __restrict__ xa, int D, int V, float scale,
                                    int buckets, int mul_prev, int mul_cur, int pos_rows, float* __restrict__ prev_state, long long SS,
                                    int write_prev, BatchMeta m) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int tok = tokens[t];
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
  const int s = m.tok_seq[t], pos = m.tok_pos[t];
  const bf16* brow = nullptr;
  if (bigram != nullptr) {
    long long row = buckets;
    if (pos > 0) {
      int prev;
      if (t > 0 && m.tok_seq[t - 1] == s) prev = tokens[t - 1];
      else prev = __float_as_int(prev_state[(long long)m.seq_slot[s] * SS]);
      prev = prev < 0 ? 0 : (prev >= V ? V - 1 : prev);
      row = ((long long)prev * mul_prev + (long long)tok * mul_cur) % buckets;
    }
    brow = bigram + row * D;
  }
  const bf16* prow = pos_tab != nullptr ? pos_tab + (long long)(pos < pos_rows ? pos : pos_rows - 1) * D : nullptr;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float v = bf2f(emb[(long long)tok * D + i]) * scale;
    if (brow != nullptr) v += bf2f(brow[i]);
    if (prow != nullptr) v += bf2f(prow[i]);
    x[(long long)t * D + i] = v;
    if (xa != nullptr) act_store<AT>(xa + (long long)t * D + i, v);
  }
  if (write_prev && bigram != nullptr) {
    __syncthreads();   // every thread of the row has read the old word (only thread-uniform reads above, but keep the order plain)
    if (threadIdx.x == 0) prev_state[(long long)m.seq_slot[s] * SS] = __int_as_float(tok);
  }
}
// the last token of every sequence of the step becomes its slot's "previous token"
__global__ void hy_prev_token_kernel(const int* __restrict__ tokens, float* __restrict__ prev_state, long long SS, int V, int n_seqs, BatchMeta m) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= n_seqs) return;
  int tok = tokens[m.seq_last[s]];
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
  prev_state[(long long)m.seq_slot[s] * SS] = __int_as_float(tok);
}

// ----------------------------------------------------------------------------- residual + norms, one block per row
// m   = s1 * m1 + s2 * m2                         (branch output; absent when m1 has no data)
// x  += m / rms(m) * (bw + bw_one)                (bw_one = 1: weight stored as an offset from one; 0: plain weight)
// hn  = x / rms(x) * (1 + nw)                     (the next reader's norm; skipped when nw == nullptr)
// xa  = x as a Linear input                       (skipped when xa == nullptr)
// plain_add: the branches are added as they are, x += s1 * m1 + s2 * m2 + m3 (no branch norm, bw unused).
// nw_mode: 0 = weight stored as an offset from one (1 + nw[i]); 1 = plain weight nw[i]; 2 = one number nw[0].
// ha  = hn as a Linear input                      (skipped when ha == nullptr)
struct RowOpArgs {
  float* x;
  LinOut m1, m2, m3;
  float s1, s2;
  const float* bw;
  float bw_one;
  const float* nw;
  float* hn;
  void* xa;
  void* ha;
  float eps;
  int D;
  int plain_add, nw_mode;
  // read by hy_row_op_ext_kernel / hy_row_op_vec_kernel only:
  int groups;       // > 1: every norm divides each of `groups` equal consecutive parts of the row by its own root mean square
  float res_mult;   // the normed branch is multiplied by this before it joins the stream
  int ext;          // the sandwich wrapper sets it when a model uses any of: groups, res_mult, plain weights, ha
  // read by hy_row_op_gated_kernel only:
  LinOut gate;      // the branch is multiplied by sigmoid(gate[t, gate_off + i]) before its norm; no data = no gate
  int gate_off;
  int bw_mode;      // branch-norm weight: 1 = plain weight bw[i]; 2 = one number bw[0]
};
#define HY_MAX_NORM_GROUPS 64
// 1 / sqrt(mean(part^2) + eps) of each part of row[0, D) into ginv: a warp per part, lanes stride the part (a fixed order,
// so the result does not depend on the launch shape).  Ends with a barrier.
__device__ __forceinline__ void hy_group_inv(const float* row, int D, int groups, float eps, float* ginv) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5, gs = D / groups;
  __syncthreads();
  for (int g = warp; g < groups; g += nw) {
    const float* p = row + (long long)g * gs;
    float ss = 0.f;
    for (int j = lane; j < gs; j += 32) ss = fmaf(p[j], p[j], ss);
    ss = warp_sum(ss);
    if (lane == 0) ginv[g] = 1.0f / sqrtf(ss / (float)gs + eps);
  }
  __syncthreads();
}
__device__ __forceinline__ float hy_norm_weight(const float* nw, int mode, int i) {
  return mode == 0 ? 1.0f + nw[i] : (mode == 1 ? nw[i] : nw[0]);
}

template <typename AT, int NT>
__global__ void __launch_bounds__(NT) hy_row_op_kernel(RowOpArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row[];
  __shared__ float red[32];
  const long long t = blockIdx.x;
  const int D = a.D;
  float* x = a.x + t * D;
  const bool branch = a.m1.f != nullptr || a.m1.h != nullptr;
  const bool two = a.m2.f != nullptr || a.m2.h != nullptr;
  if (branch && a.plain_add) {
    const bool three = a.m3.f != nullptr || a.m3.h != nullptr;
    float s2 = 0.f;
    for (int i = threadIdx.x; i < D; i += NT) {
      float b = a.s1 * lin_at(a.m1, t, i);
      if (two) b += a.s2 * lin_at(a.m2, t, i);
      if (three) b += lin_at(a.m3, t, i);
      const float v = x[i] + b;
      x[i] = v;
      row[i] = v;
      s2 += v * v;
    }
    if (a.nw == nullptr && a.xa == nullptr) return;
    s2 = block_sum<NT>(s2, red);
    if (a.nw != nullptr) {
      const float inv2 = 1.0f / sqrtf(s2 / (float)D + a.eps);
      for (int i = threadIdx.x; i < D; i += NT) {
        const float v = row[i] * inv2 * hy_norm_weight(a.nw, a.nw_mode, i);
        a.hn[t * D + i] = v;
        if (a.ha != nullptr) act_store<AT>(reinterpret_cast<AT*>(a.ha) + t * D + i, v);
      }
    }
  } else if (branch) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += NT) {
      float v = a.s1 * lin_at(a.m1, t, i);
      if (two) v += a.s2 * lin_at(a.m2, t, i);
      row[i] = v;
      ss += v * v;
    }
    ss = block_sum<NT>(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)D + a.eps);
    float s2 = 0.f;
    for (int i = threadIdx.x; i < D; i += NT) {
      const float v = x[i] + row[i] * inv * (a.bw[i] + a.bw_one);
      x[i] = v;
      row[i] = v;
      s2 += v * v;
    }
    if (a.nw == nullptr && a.xa == nullptr) return;
    s2 = block_sum<NT>(s2, red);
    if (a.nw != nullptr) {
      const float inv2 = 1.0f / sqrtf(s2 / (float)D + a.eps);
      for (int i = threadIdx.x; i < D; i += NT) a.hn[t * D + i] = row[i] * inv2 * (1.0f + a.nw[i]);
    }
  } else {
    float s2 = 0.f;
    for (int i = threadIdx.x; i < D; i += NT) {
      const float v = x[i];
      row[i] = v;
      s2 += v * v;
    }
    s2 = block_sum<NT>(s2, red);
    if (a.nw != nullptr) {
      const float inv2 = 1.0f / sqrtf(s2 / (float)D + a.eps);
      if (a.nw_mode == 0 && a.ha == nullptr) {
        for (int i = threadIdx.x; i < D; i += NT) a.hn[t * D + i] = row[i] * inv2 * (1.0f + a.nw[i]);
      } else {
        for (int i = threadIdx.x; i < D; i += NT) {
          const float v = row[i] * inv2 * hy_norm_weight(a.nw, a.nw_mode, i);
          a.hn[t * D + i] = v;
          if (a.ha != nullptr) act_store<AT>(reinterpret_cast<AT*>(a.ha) + t * D + i, v);
        }
      }
    }
  }
  if (a.xa != nullptr) {
    AT* xa = reinterpret_cast<AT*>(a.xa) + t * D;
    for (int i = threadIdx.x; i < D; i += NT) act_store<AT>(xa + i, row[i]);
  }
}

// The sandwich form with the options a design may set beside Refatar's: norms in `groups` parts, a multiplier on the normed
// branch, plain or offset weights (bw_one / nw_mode), the next reader's norm also as a Linear input (ha).
//   x += res_mult * gnorm(s1 m1 + s2 m2) * (bw + bw_one);  hn = gnorm(x) * weight(nw);  ha = hn;  xa = x
template <typename AT, int NT>
__global__ void __launch_bounds__(NT) hy_row_op_ext_kernel(RowOpArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row[];
  __shared__ float ginv[HY_MAX_NORM_GROUPS];
  const long long t = blockIdx.x;
  const int D = a.D, groups = a.groups > 1 ? a.groups : 1, gs = D / groups;
  float* x = a.x + t * D;
  const bool branch = a.m1.f != nullptr || a.m1.h != nullptr;
  const bool two = a.m2.f != nullptr || a.m2.h != nullptr;
  if (branch) {
    for (int i = threadIdx.x; i < D; i += NT) {
      float v = a.s1 * lin_at(a.m1, t, i);
      if (two) v += a.s2 * lin_at(a.m2, t, i);
      row[i] = v;
    }
    hy_group_inv(row, D, groups, a.eps, ginv);
    for (int i = threadIdx.x; i < D; i += NT) {
      const float v = x[i] + a.res_mult * (row[i] * ginv[i / gs] * (a.bw[i] + a.bw_one));
      x[i] = v;
      row[i] = v;
    }
  } else {
    for (int i = threadIdx.x; i < D; i += NT) row[i] = x[i];
  }
  if (a.nw != nullptr) {
    hy_group_inv(row, D, groups, a.eps, ginv);
    for (int i = threadIdx.x; i < D; i += NT) {
      const float v = row[i] * ginv[i / gs] * hy_norm_weight(a.nw, a.nw_mode, i);
      a.hn[t * D + i] = v;
      if (a.ha != nullptr) act_store<AT>(reinterpret_cast<AT*>(a.ha) + t * D + i, v);
    }
  }
  if (a.xa != nullptr) {
    __syncthreads();
    AT* xa = reinterpret_cast<AT*>(a.xa) + t * D;
    for (int i = threadIdx.x; i < D; i += NT) act_store<AT>(xa + i, row[i]);
  }
}

// The sandwich form for prompts whose branch is ONE bf16 matrix (the tensor-core Linear's output, no bias): the same
// arithmetic as hy_row_op_kernel with eight neighbouring channels per thread (16-byte loads of the branch, 32-byte loads and
// stores of the stream).  D, the branch's row pitch: multiples of 8.  One block of 256 threads per row.
__device__ __forceinline__ void hy_load8(const bf16* p, const float* bias, float* v);   // eight bf16 neighbours as floats (below)
__device__ __forceinline__ void hy_ld8f(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void hy_st8f(float* p, const float* v) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
// Branch-norm blocks: the sublayer read the stream itself, only its output is normed.
//   y   = m1 * sigmoid(gate)                       (gate optional)
//   x  += y / rms(y) * weight(bw)                  (bw_mode: a weight per channel or one number)
//   xa  = x as a Linear input (what the next sublayer reads);  hn = x / rms(x) * weight(nw)  (the model's last norm; nw may be nullptr)
// All of it in fp32; one block per row, the row in shared memory.
template <typename AT, int NT>
__global__ void __launch_bounds__(NT) hy_row_op_gated_kernel(RowOpArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row[];
  __shared__ float red[32];
  const long long t = blockIdx.x;
  const int D = a.D;
  float* x = a.x + t * D;
  const bool gated = a.gate.f != nullptr || a.gate.h != nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += NT) {
    float v = lin_at(a.m1, t, i);
    if (gated) v *= hy_sigmoid(lin_at(a.gate, t, a.gate_off + i));
    row[i] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum<NT>(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)D + a.eps);
  float s2 = 0.f;
  for (int i = threadIdx.x; i < D; i += NT) {
    const float v = x[i] + row[i] * inv * (a.bw_mode == 2 ? a.bw[0] : a.bw[i]);
    x[i] = v;
    row[i] = v;
    s2 = fmaf(v, v, s2);
    if (a.xa != nullptr) act_store<AT>(reinterpret_cast<AT*>(a.xa) + t * D + i, v);
  }
  if (a.nw == nullptr) return;
  s2 = block_sum<NT>(s2, red);
  const float inv2 = 1.0f / sqrtf(s2 / (float)D + a.eps);
  for (int i = threadIdx.x; i < D; i += NT) a.hn[t * D + i] = row[i] * inv2 * hy_norm_weight(a.nw, a.nw_mode, i);
}

template <typename AT> __device__ __forceinline__ void hy_st8a(AT* p, const float* v);
template <> __device__ __forceinline__ void hy_st8a<float>(float* p, const float* v) { hy_st8f(p, v); }
template <> __device__ __forceinline__ void hy_st8a<bf16>(bf16* p, const float* v) {
  *reinterpret_cast<uint4*>(p) = make_uint4(f2_to_bf2(v[0], v[1]), f2_to_bf2(v[2], v[3]), f2_to_bf2(v[4], v[5]), f2_to_bf2(v[6], v[7]));
}
// hy_row_op_gated_kernel for prompts whose branch and gate are bf16 matrices out of the tensor-core Linear: eight channels
// per thread, 16-byte loads, the new row written as the stream and as the next Linear input in one pass.  D, the pitches and
// gate_off are multiples of 8; the branch carries no bias, the gate's (fp32) is added on read.
template <typename AT>
__global__ void __launch_bounds__(256) hy_row_op_gated_vec_kernel(RowOpArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int NT = 256;
  extern __shared__ __align__(16) float row[];
  __shared__ float red[32];
  const long long t = blockIdx.x;
  const int D = a.D;
  float* x = a.x + t * D;
  const bf16* br = a.m1.h + t * a.m1.ld;
  const bool gated = a.gate.h != nullptr;
  const bf16* gr = gated ? a.gate.h + t * a.gate.ld + a.gate_off : nullptr;
  const float* gb = (gated && a.gate.bias != nullptr) ? a.gate.bias + a.gate_off : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < D; i += NT * 8) {
    float v[8];
    hy_load8(br + i, nullptr, v);
    if (gated) {
      float g[8];
      hy_load8(gr + i, gb != nullptr ? gb + i : nullptr, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] *= hy_sigmoid(g[j]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss = fmaf(v[j], v[j], ss);
    hy_st8f(row + i, v);
  }
  const float inv = 1.0f / sqrtf(block_sum<NT>(ss, red) / (float)D + a.eps);
  ss = 0.f;
  for (int i = threadIdx.x * 8; i < D; i += NT * 8) {   // a thread revisits the channels it wrote itself
    float v[8], xv[8];
    hy_ld8f(row + i, v);
    hy_ld8f(x + i, xv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      xv[j] = xv[j] + v[j] * inv * (a.bw_mode == 2 ? a.bw[0] : a.bw[i + j]);
      ss = fmaf(xv[j], xv[j], ss);
    }
    hy_st8f(x + i, xv);
    if (a.xa != nullptr) hy_st8a<AT>(reinterpret_cast<AT*>(a.xa) + t * D + i, xv);
    if (a.nw != nullptr) hy_st8f(row + i, xv);
  }
  if (a.nw == nullptr) return;
  const float inv2 = 1.0f / sqrtf(block_sum<NT>(ss, red) / (float)D + a.eps);
  for (int i = threadIdx.x * 8; i < D; i += NT * 8) {
    float v[8];
    hy_ld8f(row + i, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = v[j] * inv2 * hy_norm_weight(a.nw, a.nw_mode, i + j);
    hy_st8f(a.hn + t * D + i, v);
  }
}

template <typename AT>
__global__ void __launch_bounds__(256) hy_row_op_vec_kernel(RowOpArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int NT = 256;
  extern __shared__ __align__(16) float row[];
  __shared__ float red[32];
  __shared__ float ginv[HY_MAX_NORM_GROUPS];
  const long long t = blockIdx.x;
  const int D = a.D, groups = a.groups > 1 ? a.groups : 1, gs = D / groups;
  float* x = a.x + t * D;
  const bf16* br = a.m1.h + t * a.m1.ld;
  // branch -> row[], its norm
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < D; i += NT * 8) {
    float v[8];
    hy_load8(br + i, nullptr, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) { v[j] *= a.s1; ss = fmaf(v[j], v[j], ss); }
    hy_st8f(row + i, v);
  }
  float inv = 0.f;
  if (groups > 1) hy_group_inv(row, D, groups, a.eps, ginv);
  else inv = 1.0f / sqrtf(block_sum<NT>(ss, red) / (float)D + a.eps);
  // x += res_mult * normed branch * weight; row[] <- x
  ss = 0.f;
  for (int i = threadIdx.x * 8; i < D; i += NT * 8) {
    float v[8], xv[8], w[8];
    hy_ld8f(row + i, v);
    hy_ld8f(x + i, xv);
    hy_ld8f(a.bw + i, w);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float iv = groups > 1 ? ginv[(i + j) / gs] : inv;
      xv[j] = xv[j] + a.res_mult * (v[j] * iv * (w[j] + a.bw_one));
      ss = fmaf(xv[j], xv[j], ss);
    }
    hy_st8f(x + i, xv);
    hy_st8f(row + i, xv);
  }
  if (a.nw != nullptr) {
    if (groups > 1) hy_group_inv(row, D, groups, a.eps, ginv);
    else inv = 1.0f / sqrtf(block_sum<NT>(ss, red) / (float)D + a.eps);
    for (int i = threadIdx.x * 8; i < D; i += NT * 8) {
      float v[8];
      hy_ld8f(row + i, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = v[j] * (groups > 1 ? ginv[(i + j) / gs] : inv) * hy_norm_weight(a.nw, a.nw_mode, i + j);
      hy_st8f(a.hn + t * D + i, v);
      if (a.ha != nullptr) hy_st8a<AT>(reinterpret_cast<AT*>(a.ha) + t * D + i, v);
    }
  }
  if (a.xa != nullptr) {
    if (a.nw == nullptr) __syncthreads();
    for (int i = threadIdx.x * 8; i < D; i += NT * 8) {
      float v[8];
      hy_ld8f(row + i, v);
      hy_st8a<AT>(reinterpret_cast<AT*>(a.xa) + t * D + i, v);
    }
  }
}

// ----------------------------------------------------------------------------- causal per-channel filter
// out[t, c] = (identity ? in[t, c] : 0) + sum_j w[c, j] * in[t - (taps-1-j), c], optionally through SiLU.  Inputs of
// earlier calls come from the slot's tail (the last taps-1 inputs, oldest first); inputs before position 0 are zero.
template <typename OT>
__global__ void hy_taps_kernel(LinOut in, int col0, int C, int taps, const float* __restrict__ w, const float* __restrict__ tail,
                               long long tail_stride, BatchMeta m, int identity, int act_silu, OT* __restrict__ out, long long ld_out) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int s = m.tok_seq[row];
  const int start = s > 0 ? m.seq_last[s - 1] + 1 : 0;
  const int pos = m.tok_pos[row], pos0 = m.tok_pos[start];
  const float* tl = tail + (long long)m.seq_slot[s] * tail_stride;
  float acc = identity ? lin_at(in, row, col0 + c) : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int back = taps - 1 - j;
    const int p = pos - back;
    if (p < 0) continue;
    float v;
    if (row - back >= start) v = lin_at(in, row - back, col0 + c);
    else v = tl[(long long)(p - (pos0 - (taps - 1))) * C + c];
    acc += w[(long long)c * taps + j] * v;
  }
  if (act_silu) acc = hy_silu(acc);
  act_store<OT>(out + (long long)row * ld_out + c, acc);
}

// The same filter with the tap count known at compile time: a thread owns a channel and walks TT consecutive token rows
// with the last TAPS-1 inputs in registers, so weights and earlier inputs are read once per tile (TT = 16 for prompts; TT = 1
// gives steps of few rows a block per row).  A sequence ends where the next row belongs to another.  The window is rebuilt (earlier rows of the step, the
// slot's tail, or zeros before position 0) at the tile's first row and wherever a sequence begins.  write_tail (steps in
// which no sequence spans two tiles, e.g. one token per sequence): the thread that holds a sequence's last row also
// leaves the slot's new tail, so hy_tail_update_kernel need not run.
template <typename OT, int TAPS, int TT>
__global__ void __launch_bounds__(256) hy_taps_tile_kernel(LinOut in, int col0, int C, const float* __restrict__ w, float* __restrict__ tail,
                                                           long long tail_stride, BatchMeta m, int identity, int act_silu, int write_tail,
                                                           OT* __restrict__ out, long long ld_out, int T) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int r0 = blockIdx.x * TT;
  const int last_row = (r0 + TT < T ? r0 + TT : T) - 1;
  // most tiles lie inside one sequence (rows of a sequence are contiguous): then no row asks again
  const int s_first = m.tok_seq[r0], s_last = m.tok_seq[last_row];
  const int s_next = last_row + 1 < T ? m.tok_seq[last_row + 1] : -1;
  const bool uniform = s_first == s_last;
  float wv[TAPS];
#pragma unroll
  for (int j = 0; j < TAPS; ++j) wv[j] = w[(long long)c * TAPS + j];
  float win[TAPS];   // win[d - 1]: the input d steps back (TAPS - 1 used)
#pragma unroll
  for (int d = 0; d < TAPS; ++d) win[d] = 0.f;
#pragma unroll
  for (int i = 0; i < TT; ++i) {
    const int row = r0 + i;
    if (row > last_row) break;
    const int s = uniform ? s_first : m.tok_seq[row];
    const bool begins = !uniform && i > 0 && m.tok_seq[row - 1] != s;
    if (i == 0 || begins) {
      const float* tl = tail + (long long)m.seq_slot[s] * tail_stride;
      const int start = begins ? row : (s > 0 ? m.seq_last[s - 1] + 1 : 0);
      const int pos = m.tok_pos[row], pos0 = m.tok_pos[start];
#pragma unroll
      for (int d = 1; d < TAPS; ++d) {
        const int p = pos - d;
        float v = 0.f;
        if (p >= 0) v = row - d >= start ? lin_at(in, row - d, col0 + c) : tl[(long long)(p - (pos0 - (TAPS - 1))) * C + c];
        win[d - 1] = v;
      }
    }
    const float cur = lin_at(in, row, col0 + c);
    float acc = identity ? cur : 0.f;
#pragma unroll
    for (int j = 0; j < TAPS - 1; ++j) acc += wv[j] * win[TAPS - 2 - j];   // oldest first, as hy_taps_kernel
    acc += wv[TAPS - 1] * cur;
    if (act_silu) acc = hy_silu(acc);
    act_store<OT>(out + (long long)row * ld_out + c, acc);
#pragma unroll
    for (int d = TAPS - 1; d >= 2; --d) win[d - 1] = win[d - 2];
    win[0] = cur;
    if (write_tail && (row == last_row ? s_next != s : (!uniform && m.tok_seq[row + 1] != s))) {
      float* tl = tail + (long long)m.seq_slot[s] * tail_stride;
#pragma unroll
      for (int j = 0; j < TAPS - 1; ++j) tl[(long long)j * C + c] = win[TAPS - 2 - j];
    }
  }
}

// the slot's tail after this call: the last taps-1 inputs of the sequence, oldest first (runs after hy_taps_kernel)
__global__ void hy_tail_update_kernel(LinOut in, int col0, int C, int taps, float* __restrict__ tail, long long tail_stride, BatchMeta m) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const SeqSpan sp = seq_span(m, s);
  float* tl = tail + (long long)sp.slot * tail_stride;
  float keep[HY_MAX_TAPS];
  const int end = sp.pos0 + sp.len;
  for (int j = 0; j < taps - 1; ++j) {
    const int p = end - (taps - 1) + j;
    float v = 0.f;
    if (p >= sp.pos0) v = lin_at(in, sp.start + (p - sp.pos0), col0 + c);
    else if (p >= 0) v = tl[(long long)(p - (sp.pos0 - (taps - 1))) * C + c];
    keep[j] = v;
  }
  for (int j = 0; j < taps - 1; ++j) tl[(long long)j * C + c] = keep[j];
}

// ----------------------------------------------------------------------------- Linear for any shape
// y[T, N] (fp32) = x[T, K] w[N, K]^T + bias.  Weights bf16 row-major, accumulation fp32 (plain FMA).
// Few rows (decode): a warp per output feature streams the weight row once for all rows.
#define HY_SMALL_T 8
template <typename AT>
__global__ void __launch_bounds__(256) hy_linear_small_kernel(const AT* __restrict__ x, long long ldx, const bf16* __restrict__ w,
                                                              const float* __restrict__ bias, float* __restrict__ y, long long ldy,
                                                              int T, int N, int K) {
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (n >= N) return;
  float acc[HY_SMALL_T];
#pragma unroll
  for (int t = 0; t < HY_SMALL_T; ++t) acc[t] = 0.f;
  const bf16* wr = w + (long long)n * K;
  if ((K & 7) == 0 && (reinterpret_cast<uintptr_t>(wr) & 15) == 0) {
    for (int k = lane * 8; k < K; k += 256) {
      const uint4 u = *reinterpret_cast<const uint4*>(wr + k);
      const float2 w0 = bf2_to_f2(u.x), w1 = bf2_to_f2(u.y), w2 = bf2_to_f2(u.z), w3 = bf2_to_f2(u.w);
      const float wv[8] = {w0.x, w0.y, w1.x, w1.y, w2.x, w2.y, w3.x, w3.y};
#pragma unroll
      for (int t = 0; t < HY_SMALL_T; ++t) {
        if (t < T) {
          const AT* xr = x + (long long)t * ldx + k;
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[t] = fmaf(wv[j], act_load<AT>(xr + j), acc[t]);
        }
      }
    }
  } else {
    for (int k = lane; k < K; k += 32) {
      const float wv = bf2f(wr[k]);
#pragma unroll
      for (int t = 0; t < HY_SMALL_T; ++t)
        if (t < T) acc[t] = fmaf(wv, act_load<AT>(x + (long long)t * ldx + k), acc[t]);
    }
  }
#pragma unroll
  for (int t = 0; t < HY_SMALL_T; ++t) {
    if (t < T) {
      const float v = warp_sum(acc[t]);
      if (lane == 0) y[(long long)t * ldy + n] = v + (bias != nullptr ? bias[n] : 0.f);
    }
  }
}

// Many rows: 64 x 64 output tile per block, 16-deep k slices through shared memory, 4 x 4 outputs per thread.
template <typename AT>
__global__ void __launch_bounds__(256) hy_linear_tiled_kernel(const AT* __restrict__ x, long long ldx, const bf16* __restrict__ w,
                                                              const float* __restrict__ bias, float* __restrict__ y, long long ldy,
                                                              int T, int N, int K) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float xs[16][68];
  __shared__ float ws[16][68];
  const int t0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += 16) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = threadIdx.x + e * 256;   // 0..1023 = 64 rows x 16 k
      const int r = idx >> 4, kk = idx & 15;
      const int k = k0 + kk;
      float xv = 0.f, wv = 0.f;
      if (k < K) {
        if (t0 + r < T) xv = act_load<AT>(x + (long long)(t0 + r) * ldx + k);
        if (n0 + r < N) wv = bf2f(w[(long long)(n0 + r) * K + k]);
      }
      xs[kk][r] = xv;
      ws[kk][r] = wv;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = t0 + ty * 4 + i;
    if (t >= T) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) y[(long long)t * ldy + n] = acc[i][j] + (bias != nullptr ? bias[n] : 0.f);
    }
  }
}

// ----------------------------------------------------------------------------- gated delta rule
// Inputs per token: q, k (kv_heads x dk) and v (heads x dv) after the short filter + SiLU, in `c` [T, 2*G*dk + H*dv];
// the fused projection P also carries the read-out gate (H*dv), b (H) and a (H) columns.
// Prep, one block per token: q and k to unit length per head (q also times dk^-1/2) and their product q . k per
// q/k head, beta = sigmoid(b), decay = exp(-exp(A_log) * softplus(a + dt_bias)).
__global__ void __launch_bounds__(256) hy_delta_prep_kernel(float* __restrict__ c, long long ldc, LinOut P, int off_b, int off_a,
                                                            const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                                            float* __restrict__ beta, float* __restrict__ decay, float* __restrict__ qk,
                                                            int H, int G, int dk) {
  pdl_launch_dependents();
  pdl_wait();
  const long long t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  float* row = c + t * ldc;
  for (int g = warp; g < G; g += nw) {   // q block, then k block
    float* pq = row + (long long)g * dk;
    float* pk = row + (long long)(G + g) * dk;
    float sq = 0.f, sk = 0.f, d = 0.f;
    for (int i = lane; i < dk; i += 32) {
      const float a = pq[i], b = pk[i];
      sq = fmaf(a, a, sq); sk = fmaf(b, b, sk); d = fmaf(a, b, d);
    }
    sq = warp_sum(sq); sk = warp_sum(sk); d = warp_sum(d);
    const float cq = 1.0f / sqrtf(sq + 1e-6f) * (1.0f / sqrtf((float)dk));
    const float ck = 1.0f / sqrtf(sk + 1e-6f);
    for (int i = lane; i < dk; i += 32) { pq[i] *= cq; pk[i] *= ck; }
    if (lane == 0) qk[t * G + g] = d * cq * ck;
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    beta[t * H + h] = hy_sigmoid(lin_at(P, t, off_b + h));
    decay[t * H + h] = expf(-expf(A_log[h]) * hy_softplus(lin_at(P, t, off_a + h) + dt_bias[h]));
  }
}

// Recurrences.  Per head the state is S [dk, dv] and every value column j evolves alone:
//   delta rule: S_j <- g S_j;  u_j = beta (v_j - k . S_j);  S_j <- S_j + k u_j;  o_j = q . S_j
//               with a = k . S_j and b = q . S_j taken on the OLD column: u_j = beta (v_j - g a), o_j = g b + (q . k) u_j
//   HGRN2:      S_j <- f * S_j + (1 - f) v_j;  o_j = q . S_j      (f per row, in the k slot of the inputs)
//   general delta rule (decay w and removal rate a per row, unit key u):
//               S_j <- w * S_j - (a * u) (u . S_j) + k v_j;  o_j = r . S_j
//               with a = u . S_j and b = (r * w) . S_j on the OLD column: o_j = b - (r . (a * u)) a + (r . k) v_j
//               (five row vectors per step: r * w, u, w, a * u, k; the two scalars in the beta / decay slots)
//   lightning:  S_j <- decay S_j + k v_j;  o_j = q . S_j          (one constant decay per head)
// LPC lanes (4, 8 or 16) own one column: lane `sub` holds the rows of the 16-byte chunks sub, sub + LPC, ... (NCH chunks,
// rows beyond dk are zero), so a dot product over the rows ends in log2(LPC) shuffles and a warp carries 32 / LPC
// columns.  More lanes per column mean more blocks and shorter per-step chains (one long sequence), fewer mean fewer
// shuffles (many sequences).  The 4 warps of a block share (sequence, head) and 128 / LPC columns; the inputs of HY_TS
// steps (q, k or f, the block's v columns, and for the delta rule beta, decay and q . k) arrive in shared memory by
// cp.async, one chunk of steps ahead of the arithmetic.
// grid (n_seqs, H, ceil(dv * LPC / 128)), 128 threads; state [slot][H][dv][dk] fp32;
// dynamic shared memory 2 * HY_TS * (NV * 4 * LPC * NCH + 128 / LPC + 4) floats, NV = hy_rec_vectors(MODE) row vectors per step.
__host__ __device__ constexpr int hy_rec_vectors(int mode) { return mode == HY_REC_GDELTA ? 5 : 2; }
#define HY_TS 16
struct RecurIn {
  const float* c;        // [T, ldc] prepared inputs
  long long ldc;
  long long qoff, koff, voff;   // columns of head 0's q, k (or f) and v; heads follow at q_stride / k_stride / dv
  long long xoff[3];     // HY_REC_GDELTA: columns of head 0's decay w, removal a*u and key k (qoff: r*w, koff: unit key u)
  int q_heads;           // delta rule: heads share q / k in groups (q head = h / (H / q_heads)); others: = H
  const float *beta, *decay, *qk;   // gated delta rule: [T, H], [T, H], [T, q_heads]; HY_REC_GDELTA: beta = r.(a*u), decay = r.k, [T, H]
  const float* hdecay;   // HY_REC_LIGHTNING: [H] constant decay per head
};
__device__ __forceinline__ void hy_cp4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void hy_cp16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void hy_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void hy_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int NCH, int LPC, int MODE>
__global__ void __launch_bounds__(128) hy_recur_kernel(RecurIn in, float* __restrict__ state, long long state_stride, float* __restrict__ o,
                                                       long long ldo, BatchMeta m, int H, int dk, int dv) {
  pdl_wait();   // no early trigger: this kernel runs long on few warps, and blocks of the next kernel parked beside them slow it
  extern __shared__ __align__(16) float stg[];
  constexpr bool DELTA = MODE == HY_REC_DELTA;
  constexpr int NV = hy_rec_vectors(MODE);
  constexpr int DKP = 4 * LPC * NCH;            // padded key dim
  constexpr int HY_RC_COLS = 128 / LPC;         // columns of a block
  constexpr int VO = NV * DKP;                  // the block's value columns follow the row vectors, then the step's scalars
  constexpr int STRIDE = VO + HY_RC_COLS + 4;
  const int s = blockIdx.x, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, sub = lane & (LPC - 1);
  const int j0 = blockIdx.z * HY_RC_COLS, jl = warp * (32 / LPC) + lane / LPC, j = j0 + jl;
  const bool live = j < dv;
  const int ncv = dv - j0 < HY_RC_COLS ? dv - j0 : HY_RC_COLS;
  const SeqSpan sp = seq_span(m, s);
  const int g = h / (H / in.q_heads);
  const float* cq = in.c + in.qoff + (long long)g * dk;
  const float* ck = in.c + in.koff + (long long)g * dk;
  const float* cv = in.c + in.voff + (long long)h * dv + j0;
  const float* cx[3] = {nullptr, nullptr, nullptr};
  if (MODE == HY_REC_GDELTA) {
#pragma unroll
    for (int i = 0; i < 3; ++i) cx[i] = in.c + in.xoff[i] + (long long)g * dk;
  }
  const float hd = MODE == HY_REC_LIGHTNING ? in.hdecay[h] : 0.f;
  // 16-byte copies when every row piece starts on a 16-byte boundary
  bool al = ((in.ldc | in.qoff | in.koff | in.voff | dk | dv) & 3) == 0 && (reinterpret_cast<uintptr_t>(in.c) & 15) == 0;
  if (MODE == HY_REC_GDELTA) al = al && ((in.xoff[0] | in.xoff[1] | in.xoff[2]) & 3) == 0;
  for (int i = threadIdx.x; i < 2 * HY_TS * STRIDE; i += blockDim.x) stg[i] = 0.f;   // padding rows / columns stay zero
  float* st = state + (long long)sp.slot * state_stride + ((long long)h * dv + (live ? j : 0)) * dk;
  float S[4 * NCH];
  {
    const bool have = live && sp.pos0 > 0;
    const bool st_al = (dk & 3) == 0 && (reinterpret_cast<uintptr_t>(st) & 15) == 0;
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      const int r = (ch * LPC + sub) * 4;
      if (have && st_al && r + 3 < dk) {
        const float4 v = *reinterpret_cast<const float4*>(st + r);
        S[4 * ch] = v.x; S[4 * ch + 1] = v.y; S[4 * ch + 2] = v.z; S[4 * ch + 3] = v.w;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) S[4 * ch + e] = (have && r + e < dk) ? st[r + e] : 0.f;
      }
    }
  }
  __syncthreads();
  auto stage = [&](int t0, float* buf) {
    const int nt = sp.len - t0 < HY_TS ? sp.len - t0 : HY_TS;
    if (al) {
      const int dq = dk >> 2, per = NV * dq + (ncv >> 2);
      for (int idx = threadIdx.x; idx < nt * per; idx += blockDim.x) {
        const int ts = idx / per, u = idx - ts * per;
        const long long row = (long long)(sp.start + t0 + ts) * in.ldc;
        float* d = buf + ts * STRIDE;
        if (u < dq) hy_cp16(d + 4 * u, cq + row + 4 * u);
        else if (u < 2 * dq) hy_cp16(d + DKP + 4 * (u - dq), ck + row + 4 * (u - dq));
        else if (NV > 2 && u < NV * dq) {
          const int vi = u / dq, uu = u - vi * dq;
          hy_cp16(d + vi * DKP + 4 * uu, cx[vi - 2] + row + 4 * uu);
        } else hy_cp16(d + VO + 4 * (u - NV * dq), cv + row + 4 * (u - NV * dq));
      }
    } else {
      const int per = NV * dk + ncv;
      for (int idx = threadIdx.x; idx < nt * per; idx += blockDim.x) {
        const int ts = idx / per, u = idx - ts * per;
        const long long row = (long long)(sp.start + t0 + ts) * in.ldc;
        float* d = buf + ts * STRIDE;
        if (u < dk) hy_cp4(d + u, cq + row + u);
        else if (u < 2 * dk) hy_cp4(d + DKP + (u - dk), ck + row + (u - dk));
        else if (NV > 2 && u < NV * dk) {
          const int vi = u / dk, uu = u - vi * dk;
          hy_cp4(d + vi * DKP + uu, cx[vi - 2] + row + uu);
        } else hy_cp4(d + VO + (u - NV * dk), cv + row + (u - NV * dk));
      }
    }
    if (DELTA) {
      for (int idx = threadIdx.x; idx < nt * 3; idx += blockDim.x) {
        const int ts = idx / 3, u = idx - ts * 3;
        const long long row = sp.start + t0 + ts;
        const float* src = u == 0 ? in.beta + row * H + h : (u == 1 ? in.decay + row * H + h : in.qk + row * in.q_heads + g);
        hy_cp4(buf + ts * STRIDE + VO + HY_RC_COLS + u, src);
      }
    }
    if (MODE == HY_REC_GDELTA) {
      for (int idx = threadIdx.x; idx < nt * 2; idx += blockDim.x) {
        const int ts = idx >> 1, u = idx & 1;
        const long long row = sp.start + t0 + ts;
        hy_cp4(buf + ts * STRIDE + VO + HY_RC_COLS + u, (u == 0 ? in.beta : in.decay) + row * H + h);
      }
    }
    hy_cp_commit();
  };
  stage(0, stg);
  int cur = 0;
  for (int t0 = 0; t0 < sp.len; t0 += HY_TS, cur ^= 1) {
    const int nt = sp.len - t0 < HY_TS ? sp.len - t0 : HY_TS;
    const bool more = t0 + HY_TS < sp.len;
    if (more) { stage(t0 + HY_TS, stg + (cur ^ 1) * HY_TS * STRIDE); hy_cp_wait<1>(); }
    else hy_cp_wait<0>();
    __syncthreads();
    const float* buf = stg + cur * HY_TS * STRIDE;
    const long long orow0 = (long long)(sp.start + t0) * ldo + (long long)h * dv + j;
    auto step = [&](int ts) {
      const float* sr = buf + ts * STRIDE;
      const float v = sr[VO + jl];
      if (MODE == HY_REC_GDELTA) {
        float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch) {
          const int r = (ch * LPC + sub) * 4;
          const float4 q4 = *reinterpret_cast<const float4*>(sr + r);
          const float4 u4 = *reinterpret_cast<const float4*>(sr + DKP + r);
          a0 = fmaf(u4.x, S[4 * ch], a0); a1 = fmaf(u4.y, S[4 * ch + 1], a1);
          a0 = fmaf(u4.z, S[4 * ch + 2], a0); a1 = fmaf(u4.w, S[4 * ch + 3], a1);
          b0 = fmaf(q4.x, S[4 * ch], b0); b1 = fmaf(q4.y, S[4 * ch + 1], b1);
          b0 = fmaf(q4.z, S[4 * ch + 2], b0); b1 = fmaf(q4.w, S[4 * ch + 3], b1);
        }
        float a = a0 + a1, b = b0 + b1;
#pragma unroll
        for (int off = 1; off < LPC; off <<= 1) {
          a += __shfl_xor_sync(0xffffffffu, a, off);
          b += __shfl_xor_sync(0xffffffffu, b, off);
        }
        const float ra = sr[VO + HY_RC_COLS], rk = sr[VO + HY_RC_COLS + 1];
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch) {
          const int r = (ch * LPC + sub) * 4;
          const float4 w4 = *reinterpret_cast<const float4*>(sr + 2 * DKP + r);
          const float4 e4 = *reinterpret_cast<const float4*>(sr + 3 * DKP + r);
          const float4 k4 = *reinterpret_cast<const float4*>(sr + 4 * DKP + r);
          S[4 * ch] = fmaf(k4.x, v, fmaf(w4.x, S[4 * ch], -e4.x * a));
          S[4 * ch + 1] = fmaf(k4.y, v, fmaf(w4.y, S[4 * ch + 1], -e4.y * a));
          S[4 * ch + 2] = fmaf(k4.z, v, fmaf(w4.z, S[4 * ch + 2], -e4.z * a));
          S[4 * ch + 3] = fmaf(k4.w, v, fmaf(w4.w, S[4 * ch + 3], -e4.w * a));
        }
        if (sub == 0 && live) o[orow0 + (long long)ts * ldo] = fmaf(rk, v, fmaf(-ra, a, b));
      } else if (MODE == HY_REC_LIGHTNING) {
        float b0 = 0.f, b1 = 0.f;
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch) {
          const int r = (ch * LPC + sub) * 4;
          const float4 q4 = *reinterpret_cast<const float4*>(sr + r);
          const float4 k4 = *reinterpret_cast<const float4*>(sr + DKP + r);
          S[4 * ch] = fmaf(hd, S[4 * ch], k4.x * v);
          S[4 * ch + 1] = fmaf(hd, S[4 * ch + 1], k4.y * v);
          S[4 * ch + 2] = fmaf(hd, S[4 * ch + 2], k4.z * v);
          S[4 * ch + 3] = fmaf(hd, S[4 * ch + 3], k4.w * v);
          b0 = fmaf(q4.x, S[4 * ch], b0); b1 = fmaf(q4.y, S[4 * ch + 1], b1);
          b0 = fmaf(q4.z, S[4 * ch + 2], b0); b1 = fmaf(q4.w, S[4 * ch + 3], b1);
        }
        float b = b0 + b1;
#pragma unroll
        for (int off = 1; off < LPC; off <<= 1) b += __shfl_xor_sync(0xffffffffu, b, off);
        if (sub == 0 && live) o[orow0 + (long long)ts * ldo] = b;
      } else if (DELTA) {
        float kv[4 * NCH];
        float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch) {
          const int r = (ch * LPC + sub) * 4;
          const float4 q4 = *reinterpret_cast<const float4*>(sr + r);
          const float4 k4 = *reinterpret_cast<const float4*>(sr + DKP + r);
          kv[4 * ch] = k4.x; kv[4 * ch + 1] = k4.y; kv[4 * ch + 2] = k4.z; kv[4 * ch + 3] = k4.w;
          a0 = fmaf(k4.x, S[4 * ch], a0); a1 = fmaf(k4.y, S[4 * ch + 1], a1);
          a0 = fmaf(k4.z, S[4 * ch + 2], a0); a1 = fmaf(k4.w, S[4 * ch + 3], a1);
          b0 = fmaf(q4.x, S[4 * ch], b0); b1 = fmaf(q4.y, S[4 * ch + 1], b1);
          b0 = fmaf(q4.z, S[4 * ch + 2], b0); b1 = fmaf(q4.w, S[4 * ch + 3], b1);
        }
        float a = a0 + a1, b = b0 + b1;
#pragma unroll
        for (int off = 1; off < LPC; off <<= 1) {
          a += __shfl_xor_sync(0xffffffffu, a, off);
          b += __shfl_xor_sync(0xffffffffu, b, off);
        }
        const float be = sr[VO + HY_RC_COLS], gd = sr[VO + HY_RC_COLS + 1], qk = sr[VO + HY_RC_COLS + 2];
        const float u = be * (v - gd * a);
#pragma unroll
        for (int i = 0; i < 4 * NCH; ++i) S[i] = fmaf(kv[i], u, gd * S[i]);
        if (sub == 0 && live) o[orow0 + (long long)ts * ldo] = fmaf(qk, u, gd * b);
      } else {
        float b0 = 0.f, b1 = 0.f;
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch) {
          const int r = (ch * LPC + sub) * 4;
          const float4 q4 = *reinterpret_cast<const float4*>(sr + r);
          const float4 f4 = *reinterpret_cast<const float4*>(sr + DKP + r);
          S[4 * ch] = fmaf(f4.x, S[4 * ch], (1.0f - f4.x) * v);
          S[4 * ch + 1] = fmaf(f4.y, S[4 * ch + 1], (1.0f - f4.y) * v);
          S[4 * ch + 2] = fmaf(f4.z, S[4 * ch + 2], (1.0f - f4.z) * v);
          S[4 * ch + 3] = fmaf(f4.w, S[4 * ch + 3], (1.0f - f4.w) * v);
          b0 = fmaf(q4.x, S[4 * ch], b0); b1 = fmaf(q4.y, S[4 * ch + 1], b1);
          b0 = fmaf(q4.z, S[4 * ch + 2], b0); b1 = fmaf(q4.w, S[4 * ch + 3], b1);
        }
        float b = b0 + b1;
#pragma unroll
        for (int off = 1; off < LPC; off <<= 1) b += __shfl_xor_sync(0xffffffffu, b, off);
        if (sub == 0 && live) o[orow0 + (long long)ts * ldo] = b;
      }
    };
    // full chunks: unrolled, so that the loads and reductions of neighbouring steps overlap (HGRN2's steps depend on one
    // another through a single FMA per row; the delta rule's through the whole a -> u -> S chain, so less is gained)
    if (nt == HY_TS) {
#pragma unroll 4
      for (int ts = 0; ts < HY_TS; ++ts) step(ts);
    } else {
      for (int ts = 0; ts < nt; ++ts) step(ts);
    }
    __syncthreads();   // the buffer is refilled by the next iteration's copies
  }
  if (live) {
    const bool st_al = (dk & 3) == 0 && (reinterpret_cast<uintptr_t>(st) & 15) == 0;
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      const int r = (ch * LPC + sub) * 4;
      if (st_al && r + 3 < dk) {
        *reinterpret_cast<float4*>(st + r) = make_float4(S[4 * ch], S[4 * ch + 1], S[4 * ch + 2], S[4 * ch + 3]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (r + e < dk) st[r + e] = S[4 * ch + e];
      }
    }
  }
}

// ----------------------------------------------------------------------------- HGRN2
// Prep: q = silu(.), f = lower + (1 - lower) sigmoid(.), v copied, into one fp32 row [q | f | v].  grid (T, ceil(n / 256)).
__global__ void hy_hgrn_prep_kernel(LinOut P, int off_q, int off_f, int off_v, const float* __restrict__ lower, float* __restrict__ c,
                                    long long ldc, int HK, int HV) {
  pdl_launch_dependents();
  pdl_wait();
  const long long t = blockIdx.x;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= 2 * HK + HV) return;
  float v;
  if (i < HK) v = hy_silu(lin_at(P, t, off_q + i));
  else if (i < 2 * HK) {
    const float lo = lower[i - HK];
    v = lo + (1.0f - lo) * hy_sigmoid(lin_at(P, t, off_f + i - HK));
  } else v = lin_at(P, t, off_v + i - 2 * HK);
  c[t * ldc + i] = v;
}

// The recurrence itself runs in hy_recur_kernel<., false> above: f sits where the delta rule has k.

// ----------------------------------------------------------------------------- per-head RMS norm (+ SiLU gate) of a read-out
// out[t, h*dv + j] = scale * o / rms_over_dv(o) * w[h * w_hstride + j] * (gate ? act(P[t, off_gate + h*dv + j]) : 1)
// w_hstride: 0 = one weight vector for all heads, dv = a vector per head; gate_sigmoid: 0 = SiLU gate, 1 = sigmoid gate.
// H = 1 with dv = all heads' size norms the concatenated read-out as one vector.
template <typename AT>
__global__ void __launch_bounds__(256) hy_head_norm_kernel(const float* __restrict__ o, long long ldo, const float* __restrict__ w,
                                                           LinOut P, int off_gate, float eps, float scale, AT* __restrict__ out,
                                                           long long ld_out, int H, int dv, int w_hstride, int gate_sigmoid) {
  pdl_launch_dependents();
  pdl_wait();
  const long long t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int h = blockIdx.y * nw + warp; h < H; h += nw * gridDim.y) {
    const float* p = o + t * ldo + (long long)h * dv;
    float ss = 0.f;
    for (int j = lane; j < dv; j += 32) ss += p[j] * p[j];
    ss = warp_sum(ss);
    const float inv = scale / sqrtf(ss / (float)dv + eps);
    for (int j = lane; j < dv; j += 32) {
      float v = p[j] * inv * w[(long long)h * w_hstride + j];
      if (off_gate >= 0) {
        const float gz = lin_at(P, t, off_gate + h * dv + j);
        v *= gate_sigmoid ? hy_sigmoid(gz) : hy_silu(gz);
      }
      act_store<AT>(out + t * ld_out + (long long)h * dv + j, v);
    }
  }
}

// ----------------------------------------------------------------------------- windowed softmax attention
// Paged pools [n_pages][G][page_tokens][d] of KT (bf16 serving, float in the all-fp32 mode).
template <typename KT>
__global__ void hy_kv_append_kernel(LinOut P, int off_k, int off_v, KT* __restrict__ k_pool, KT* __restrict__ v_pool, BatchMeta m,
                                    int G, int dk, int dv) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int s = m.tok_seq[row], pos = m.tok_pos[row];
  const int page = m.page_table[(long long)m.seq_slot[s] * m.max_pages + pos / m.page_tokens];
  const int in_page = pos % m.page_tokens;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < G * (dk + dv); i += blockDim.x * gridDim.y) {
    if (i < G * dk) {
      const int g = i / dk, d = i - g * dk;
      act_store<KT>(k_pool + (((long long)page * G + g) * m.page_tokens + in_page) * dk + d, lin_at(P, row, off_k + i));
    } else {
      const int i2 = i - G * dk;
      const int g = i2 / dv, d = i2 - g * dv;
      act_store<KT>(v_pool + (((long long)page * G + g) * m.page_tokens + in_page) * dv + d, lin_at(P, row, off_v + i2));
    }
  }
}

// q . k for one key row; 16-byte loads when the row length allows (rows then start on 16-byte boundaries)
template <typename KT> __device__ __forceinline__ float hy_dot_row(const float* __restrict__ q, const KT* __restrict__ kr, int dk);
template <> __device__ __forceinline__ float hy_dot_row<float>(const float* __restrict__ q, const float* __restrict__ kr, int dk) {
  float d = 0.f;
  if ((dk & 3) == 0) {
    for (int i = 0; i < dk; i += 4) {
      const float4 k4 = *reinterpret_cast<const float4*>(kr + i);
      const float4 q4 = *reinterpret_cast<const float4*>(q + i);
      d = fmaf(q4.x, k4.x, d); d = fmaf(q4.y, k4.y, d); d = fmaf(q4.z, k4.z, d); d = fmaf(q4.w, k4.w, d);
    }
  } else {
    for (int i = 0; i < dk; ++i) d = fmaf(q[i], kr[i], d);
  }
  return d;
}
__device__ __forceinline__ float hy_dot8(const float* __restrict__ q, const uint4 u, float d) {
  const float2 a = bf2_to_f2(u.x), b = bf2_to_f2(u.y), c = bf2_to_f2(u.z), e = bf2_to_f2(u.w);
  const float4 q0 = *reinterpret_cast<const float4*>(q), q1 = *reinterpret_cast<const float4*>(q + 4);
  d = fmaf(q0.x, a.x, d); d = fmaf(q0.y, a.y, d); d = fmaf(q0.z, b.x, d); d = fmaf(q0.w, b.y, d);
  d = fmaf(q1.x, c.x, d); d = fmaf(q1.y, c.y, d); d = fmaf(q1.z, e.x, d); d = fmaf(q1.w, e.y, d);
  return d;
}
template <> __device__ __forceinline__ float hy_dot_row<bf16>(const float* __restrict__ q, const bf16* __restrict__ kr, int dk) {
  float d = 0.f;
  if ((dk & 7) == 0) {
    int i = 0;
    for (; i + 32 <= dk; i += 32) {   // four 16-byte loads in flight
      const uint4 u0 = *reinterpret_cast<const uint4*>(kr + i), u1 = *reinterpret_cast<const uint4*>(kr + i + 8);
      const uint4 u2 = *reinterpret_cast<const uint4*>(kr + i + 16), u3 = *reinterpret_cast<const uint4*>(kr + i + 24);
      float d1 = hy_dot8(q + i + 8, u1, 0.f), d2 = hy_dot8(q + i + 16, u2, 0.f), d3 = hy_dot8(q + i + 24, u3, 0.f);
      d = hy_dot8(q + i, u0, d);
      d += (d1 + d2) + d3;
    }
    for (; i < dk; i += 8) d = hy_dot8(q + i, *reinterpret_cast<const uint4*>(kr + i), d);
  } else {
    for (int i = 0; i < dk; ++i) d = fmaf(q[i], bf2f(kr[i]), d);
  }
  return d;
}

// rows that need not start on a 16-byte boundary
template <typename KT> __device__ __forceinline__ float hy_dot_row_any(const float* __restrict__ q, const KT* __restrict__ kr, int dk) {
  float d = 0.f;
  for (int i = 0; i < dk; ++i) d = fmaf(q[i], act_load<KT>(kr + i), d);
  return d;
}

// q (bias added) and the output gate of the attention heads as one bf16 row [q | gate] per token: what the tcgen05 attention
// reads when the projection came back as split-K planes (steps of few rows).  grid (T, ceil((nq + ng) / 256)).
__global__ void hy_qg_pack_kernel(LinOut P, int off_q, int nq, int off_g, int ng, bf16* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const long long t = blockIdx.x;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= nq + ng) return;
  out[t * (nq + ng) + i] = f2bf(lin_at(P, t, i < nq ? off_q + i : off_g + (i - nq)));
}

// One block per (token, query head); its warps split the visible keys 32 at a time.  Query i sees key j when j <= i and
// (i - j < window or j < keep_first): the kept first keys, then the window.  In a 32-key tile a lane scores one key (fp32
// dot with the query in shared memory), the warp does the online softmax, then lanes own value channels for the weighted
// sum; at the end warp 0 merges the warps' (max, sum, accumulator) triples.  No rotation: positions enter through the
// mask only.  The epilogue multiplies by sigmoid(gate column) and `out_scale`.
// dv <= 32 * NACC (NACC = 8 or 16 value channels per lane).  Key / value rows of the pools are ldk / ldv elements apart
// (ldk = dk, ldv = dv for separate pools; a value that is the head of its key row reads the key pool with ldv = ldk).
// Dynamic shared memory: (dk rounded up to 4) + warps * (2 + dv) floats.
// AttnOpt: what the rotary-position attention adds.  sink (per head, or nullptr): exp(sink_h) joins the softmax
// denominator, with no key and no value.  softcap > 0: score <- cap * tanh(score / cap) (after the scale).  v_heads: value
// heads per page of the value pool; 1 while G > 1 means a value row holds every key head's values side by side
// ([page][token][G * dv], dv here = that whole width), so that one query head's weights meet all of them.
// v_chunk > 0: block z handles value channels [z * v_chunk, (z + 1) * v_chunk) of the row (rows wider than the 512 channels a
// block's lanes can carry; every block recomputes the scores).
// r1 / r2 (per head, both or neither): r1[h] * ln(1 + r2[h] * (query position - key position)) is taken off the scaled score.
struct AttnOpt {
  const float* sink;
  float softcap;
  int v_heads;
  int v_chunk;
  const float* r1;
  const float* r2;
};
template <typename KT, typename AT, int NACC>
__global__ void __launch_bounds__(512) hy_attn_window_kernel(LinOut P, int off_q, int off_gate, const KT* __restrict__ k_pool,
                                                             const KT* __restrict__ v_pool, BatchMeta m, int H, int G, int dk, int dv,
                                                             int ldk, int ldv, int window, int keep_first, float scale, float out_scale,
                                                             AT* __restrict__ out, long long ld_out, AttnOpt opt) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float qsm[];
  const int row = blockIdx.x, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int dv_full = dv;
  int voff = 0;
  if (opt.v_chunk > 0) {
    voff = (int)blockIdx.z * opt.v_chunk;
    dv = dv_full - voff < opt.v_chunk ? dv_full - voff : opt.v_chunk;
    v_pool += voff;
  }
  float* q = qsm;
  float* part = qsm + ((dk + 3) & ~3);   // per warp: max, sum, acc[dv]
  for (int i = threadIdx.x; i < dk; i += blockDim.x) q[i] = lin_at(P, row, off_q + h * dk + i) * scale;
  __syncthreads();
  const int g = h / (H / G);
  const int s = m.tok_seq[row], pos = m.tok_pos[row];
  const int* pages = m.page_table + (long long)m.seq_slot[s] * m.max_pages;
  const int lo = pos - window + 1 > 0 ? pos - window + 1 : 0;
  const int n_first = keep_first < lo ? keep_first : lo;   // kept keys that the window does not already cover
  const int n_vis = n_first + (pos - lo + 1);
  float mx = -INFINITY, l = 0.f;
  float acc[NACC];
#pragma unroll
  for (int c = 0; c < NACC; ++c) acc[c] = 0.f;
  // even dv: a lane owns channel pairs (2 * (lane + 32 c), + 1), c < 4, and takes four keys per round so that their value
  // loads are in flight together; odd dv: a lane owns channels lane + 32 c, one key per round
  const bool pairs = ((dv | ldv) & 1) == 0;
  for (int base = warp * 32; base < n_vis; base += nw * 32) {
    const int idx = base + lane;
    float sc = -INFINITY;
    long long prow = 0;
    if (idx < n_vis) {
      const int kp = idx < n_first ? idx : lo + (idx - n_first);
      const long long pg = pages[kp / m.page_tokens];
      const int ip = kp % m.page_tokens;
      const long long krow = (pg * G + g) * m.page_tokens + ip;
      prow = opt.v_heads == G ? krow : pg * m.page_tokens + ip;   // the value row (shared with the other lanes below)
      sc = (ldk & 7) == 0 ? hy_dot_row<KT>(q, k_pool + krow * ldk, dk) : hy_dot_row_any<KT>(q, k_pool + krow * ldk, dk);
      if (opt.softcap > 0.f) sc = opt.softcap * tanhf(sc / opt.softcap);
      if (opt.r1 != nullptr) sc -= opt.r1[h] * log1pf(opt.r2[h] * (float)(pos - kp));
    }
    const float tmax = warp_max(sc);
    const float nm = fmaxf(mx, tmax);
    const float corr = expf(mx - nm);   // mx = -inf on the first tile: exp(-inf) = 0
    const float p = idx < n_vis ? expf(sc - nm) : 0.f;
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int c = 0; c < NACC; ++c) acc[c] *= corr;
    mx = nm;
    const int cnt = n_vis - base < 32 ? n_vis - base : 32;
    if (pairs) {
      for (int jj = 0; jj < cnt; jj += 4) {   // lanes past cnt hold p = 0 and row 0 of the pool (finite values)
        float pj[4];
        float2 vv[4][NACC / 2];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          pj[u] = __shfl_sync(0xffffffffu, p, jj + u);
          const long long pr = __shfl_sync(0xffffffffu, prow, jj + u);
          const KT* vr = v_pool + pr * ldv;
#pragma unroll
          for (int c = 0; c < NACC / 2; ++c) {
            const int d = 2 * (lane + 32 * c);
            vv[u][c] = (64 * c < dv && d < dv) ? act_load2<KT>(vr + d) : make_float2(0.f, 0.f);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int c = 0; c < NACC / 2; ++c) {
            if (64 * c >= dv) continue;
            acc[2 * c] = fmaf(pj[u], vv[u][c].x, acc[2 * c]);
            acc[2 * c + 1] = fmaf(pj[u], vv[u][c].y, acc[2 * c + 1]);
          }
      }
    } else {
      for (int jj = 0; jj < cnt; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, p, jj);
        const long long pr = __shfl_sync(0xffffffffu, prow, jj);
        const KT* vr = v_pool + pr * ldv;
#pragma unroll
        for (int c = 0; c < NACC; ++c) {
          const int d = lane + 32 * c;
          if (d < dv) acc[c] = fmaf(pj, act_load<KT>(vr + d), acc[c]);
        }
      }
    }
  }
  float* mine = part + (long long)warp * (2 + dv);
  if (lane == 0) { mine[0] = mx; mine[1] = l; }
  if (pairs) {
#pragma unroll
    for (int c = 0; c < NACC / 2; ++c) {
      const int d = 2 * (lane + 32 * c);
      if (d < dv) { mine[2 + d] = acc[2 * c]; mine[3 + d] = acc[2 * c + 1]; }
    }
  } else {
#pragma unroll
    for (int c = 0; c < NACC; ++c) {
      const int d = lane + 32 * c;
      if (d < dv) mine[2 + d] = acc[c];
    }
  }
  __syncthreads();
  if (warp != 0) return;
  float M = -INFINITY;
  for (int w = 0; w < nw; ++w) M = fmaxf(M, part[(long long)w * (2 + dv)]);
  float L = 0.f;
  if (opt.sink != nullptr) {
    const float sk = opt.sink[h];
    M = fmaxf(M, sk);
    L = expf(sk - M);
  }
#pragma unroll
  for (int c = 0; c < NACC; ++c) acc[c] = 0.f;
  for (int w = 0; w < nw; ++w) {
    const float* pw = part + (long long)w * (2 + dv);
    const float f = expf(pw[0] - M);     // a warp without keys holds max = -inf: weight 0
    L += pw[1] * f;
#pragma unroll
    for (int c = 0; c < NACC; ++c) {
      const int d = lane + 32 * c;
      if (d < dv) acc[c] = fmaf(pw[2 + d], f, acc[c]);
    }
  }
  const float inv = out_scale / L;
#pragma unroll
  for (int c = 0; c < NACC; ++c) {
    const int d = lane + 32 * c;
    if (d < dv) {
      float v = acc[c] * inv;
      if (off_gate >= 0) v *= hy_sigmoid(lin_at(P, row, off_gate + h * dv_full + voff + d));
      act_store<AT>(out + (long long)row * ld_out + (long long)h * dv_full + voff + d, v);
    }
  }
}

// ----------------------------------------------------------------------------- whole-projection q / k norms, query temperature, cache append
// Attention without rotation whose queries and keys are RMS-normed over the WHOLE projection (all heads of a token as one
// vector, a weight per channel; qn / kn nullptr = no norm) and whose queries carry a temperature that grows with the
// position, q *= 1 + coef * ln(floor((pos + 1) / every) + 1) (every = 0: none).  One block per token, the token's q and k
// channels in shared memory ((H + G) * dk floats):
//   qa[t]  (fp32, rows of H * dk)  and, when asked, qg[t] (bf16, for a tensor-core kernel) = the finished queries
//   k_pool [page][G][token][dk]    = the finished keys
//   v_pool [page][G][token][dv]    = P[t, off_v ...]: the value projection, or with off_v = off_k (dv = dk) the keys as they were
//                                    projected, before the norm
// Everything after the projection is fp32.  qa may be nullptr (a tensor-core kernel reads qg instead).  NT threads: 256 for
// prompts, 1024 in steps of few rows, where the reads of the projection's split-K planes are what takes the time.
template <typename KT, int NT>
__global__ void __launch_bounds__(NT) hy_qk_prep_kernel(LinOut P, int off_q, int off_k, int off_v, int H, int G, int dk, int dv,
                                                         const float* __restrict__ qn, const float* __restrict__ kn, float eps,
                                                         float temp_coef, int temp_every, float* __restrict__ qa, bf16* __restrict__ qg,
                                                         KT* __restrict__ k_pool, KT* __restrict__ v_pool, BatchMeta m) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float qk[];
  __shared__ float red[32];
  const int row = blockIdx.x;
  const int nq = H * dk, nk = G * dk, nv = G * dv;
  const int s = m.tok_seq[row], pos = m.tok_pos[row];
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < nq; i += NT) { const float v = lin_at(P, row, off_q + i); qk[i] = v; sq = fmaf(v, v, sq); }
  for (int i = threadIdx.x; i < nk; i += NT) { const float v = lin_at(P, row, off_k + i); qk[nq + i] = v; sk = fmaf(v, v, sk); }
  float qs = 1.f, ks = 1.f;
  if (qn != nullptr) qs = 1.0f / sqrtf(block_sum<NT>(sq, red) / (float)nq + eps);
  if (kn != nullptr) ks = 1.0f / sqrtf(block_sum<NT>(sk, red) / (float)nk + eps);
  __syncthreads();
  const float temp = temp_every > 0 ? 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f) : 1.0f;
  for (int i = threadIdx.x; i < nq; i += NT) {
    const float v = qn != nullptr ? qk[i] * qs * qn[i] * temp : qk[i] * temp;
    if (qa != nullptr) qa[(long long)row * nq + i] = v;
    if (qg != nullptr) qg[(long long)row * nq + i] = f2bf(v);
  }
  const long long pg = m.page_table[(long long)m.seq_slot[s] * m.max_pages + pos / m.page_tokens];
  const int ip = pos % m.page_tokens;
  for (int i = threadIdx.x; i < nk; i += NT) {
    const int g = i / dk, c = i - g * dk;
    const float v = kn != nullptr ? qk[nq + i] * ks * kn[i] : qk[nq + i];
    act_store<KT>(k_pool + ((pg * G + g) * m.page_tokens + ip) * dk + c, v);
  }
  for (int i = threadIdx.x; i < nv; i += NT) {
    const int g = i / dv, c = i - g * dv;
    const float v = off_v == off_k ? qk[nq + i] : lin_at(P, row, off_v + i);
    act_store<KT>(v_pool + ((pg * G + g) * m.page_tokens + ip) * dv + c, v);
  }
}

// The same arithmetic on 16-byte accesses, for prompts whose projection came back as ONE bf16 matrix and whose pools are bf16:
// eight neighbouring channels per thread.  off_q, off_k, off_v, dk, dv and the projection's row pitch are multiples of 8;
// the finished queries leave as bf16 rows (qg).  One block of 256 threads per token.
__device__ __forceinline__ uint4 hy_pack8(const float* y);   // eight floats as bf16 neighbours (below)
__global__ void __launch_bounds__(256) hy_qk_prep_vec_kernel(const bf16* __restrict__ P, long long ldp, const float* __restrict__ bias, int off_q, int off_k,
                                                             int off_v, int H, int G, int dk, int dv, const float* __restrict__ qn,
                                                             const float* __restrict__ kn, float eps, float temp_coef, int temp_every,
                                                             bf16* __restrict__ qg, bf16* __restrict__ k_pool, bf16* __restrict__ v_pool, BatchMeta m) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float qk[];
  __shared__ float red[32];
  const int row = blockIdx.x;
  const int nq = H * dk, nk = G * dk, nv = G * dv;
  const int s = m.tok_seq[row], pos = m.tok_pos[row];
  const bf16* prow = P + (long long)row * ldp;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x * 8; i < nq + nk; i += 256 * 8) {
    const int col = i < nq ? off_q + i : off_k + (i - nq);
    float v[8];
    hy_load8(prow + col, bias != nullptr ? bias + col : nullptr, v);
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) ss = fmaf(v[j], v[j], ss);
    if (i < nq) sq += ss; else sk += ss;
    hy_st8f(qk + i, v);
  }
  float qs = 1.f, ks = 1.f;
  if (qn != nullptr) qs = 1.0f / sqrtf(block_sum<256>(sq, red) / (float)nq + eps);
  if (kn != nullptr) ks = 1.0f / sqrtf(block_sum<256>(sk, red) / (float)nk + eps);
  __syncthreads();
  const float temp = temp_every > 0 ? 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f) : 1.0f;
  const long long pg = m.page_table[(long long)m.seq_slot[s] * m.max_pages + pos / m.page_tokens];
  const int ip = pos % m.page_tokens;
  for (int i = threadIdx.x * 8; i < nq + nk; i += 256 * 8) {   // a thread revisits the channels it wrote itself
    float v[8], w[8];
    hy_ld8f(qk + i, v);
    if (i < nq) {
      if (qn != nullptr) {
        hy_ld8f(qn + i, w);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = v[j] * qs * w[j] * temp;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] *= temp;
      }
      *reinterpret_cast<uint4*>(qg + (long long)row * nq + i) = hy_pack8(v);
    } else {
      const int ik = i - nq, g = ik / dk, c = ik - g * dk;
      if (off_v == off_k)   // the values are the keys as projected
        *reinterpret_cast<uint4*>(v_pool + ((pg * G + g) * m.page_tokens + ip) * dv + c) = hy_pack8(v);
      if (kn != nullptr) {
        hy_ld8f(kn + ik, w);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = v[j] * ks * w[j];
      }
      *reinterpret_cast<uint4*>(k_pool + ((pg * G + g) * m.page_tokens + ip) * dk + c) = hy_pack8(v);
    }
  }
  if (off_v != off_k)
    for (int i = threadIdx.x * 8; i < nv; i += 256 * 8) {
      const int g = i / dv, c = i - g * dv;
      float v[8];
      hy_load8(prow + off_v + i, bias != nullptr ? bias + off_v + i : nullptr, v);
      *reinterpret_cast<uint4*>(v_pool + ((pg * G + g) * m.page_tokens + ip) * dv + c) = hy_pack8(v);
    }
}

// ----------------------------------------------------------------------------- rotary positions, value blending, head mixing
// Rotation of the first `dims` entries of a head: entry pairs (i, i + dims/2) (half = 1) or (2i, 2i + 1) (half = 0);
// (u, v) -> (u c - v s, v c + u s) with c, s = mult * cos / sin(pos * freq[i]).  The angle is formed in double and reduced
// to [-pi, pi] there, so that its error does not grow with the position.
#define HY_MAX_ROT_PAIRS 256   // rotating pairs per head (key dim <= 512)
struct RotArgs {
  const double* freq;   // [dims / 2]
  int dims, half;
  float mult;
};
__device__ __forceinline__ void hy_rot_cs(const RotArgs& r, int pos, int i, float* c, float* s) {
  double a = (double)pos * r.freq[i];
  a -= 6.283185307179586 * rint(a * 0.15915494309189535);
  sincosf((float)a, s, c);
  *c *= r.mult;
  *s *= r.mult;
}
// One token row of an XB_MIX_SOFTMAX layer after its input projection P = [q | k | v | ...]: rotated queries -> qa (fp32
// [T, H * dk], or bf16 q16 when given: what the tensor-core attention reads), rotated keys -> the key pool, values -> the
// value pool.  vmode 1: the values are also left in vfirst
// ([T, G * dv] fp32) for later layers of the step; vmode 2: v <- (1 - l) v + l vfirst with l = vmix[0] before they are
// cached.  v_all: a value row holds all G heads ([page][token][G * dv]) instead of [page][G][token][dv].
// A thread owns a rotating pair or one entry that does not turn.  grid (T, ceil(units / 256)).
template <typename KT>
__global__ void __launch_bounds__(256) hy_rope_append_kernel(LinOut P, int off_q, int off_k, int off_v, int H, int G, int dk, int dv,
                                                             RotArgs r, float* __restrict__ qa, bf16* __restrict__ q16, KT* __restrict__ k_pool,
                                                             KT* __restrict__ v_pool, int v_all, const float* __restrict__ vmix,
                                                             float* __restrict__ vfirst, int vmode, BatchMeta m) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int s = m.tok_seq[row], pos = m.tok_pos[row];
  const long long page = m.page_table[(long long)m.seq_slot[s] * m.max_pages + pos / m.page_tokens];
  const int in_page = pos % m.page_tokens;
  const int hp = r.dims >> 1, per = dk - hp;   // units of one query / key head
  const int n_qk = (H + G) * per, total = n_qk + G * dv;
  // every head of the token turns by the same angles: cos / sin of the pairs once per block
  __shared__ float cs_tab[2 * HY_MAX_ROT_PAIRS];
  for (int j = threadIdx.x; j < hp; j += blockDim.x) hy_rot_cs(r, pos, j, &cs_tab[2 * j], &cs_tab[2 * j + 1]);
  __syncthreads();
  for (int u = blockIdx.y * blockDim.x + threadIdx.x; u < total; u += blockDim.x * gridDim.y) {
    if (u < n_qk) {
      const int hd = u / per, j = u - hd * per;
      const bool is_q = hd < H;
      const int h = is_q ? hd : hd - H;
      const int src = (is_q ? off_q : off_k) + h * dk;
      const long long qi = (long long)row * H * dk + (long long)h * dk;
      KT* ko = k_pool + ((page * G + h) * m.page_tokens + in_page) * dk;
      if (j < hp) {
        const int d0 = r.half ? j : 2 * j, d1 = r.half ? j + hp : 2 * j + 1;
        const float a = lin_at(P, row, src + d0), b = lin_at(P, row, src + d1);
        const float c = cs_tab[2 * j], sn = cs_tab[2 * j + 1];
        const float y0 = a * c - b * sn, y1 = b * c + a * sn;
        if (!is_q) { act_store<KT>(ko + d0, y0); act_store<KT>(ko + d1, y1); }
        else if (q16 != nullptr) { q16[qi + d0] = f2bf(y0); q16[qi + d1] = f2bf(y1); }
        else { qa[qi + d0] = y0; qa[qi + d1] = y1; }
      } else {
        const int d = r.dims + (j - hp);
        const float a = lin_at(P, row, src + d);
        if (!is_q) act_store<KT>(ko + d, a);
        else if (q16 != nullptr) q16[qi + d] = f2bf(a);
        else qa[qi + d] = a;
      }
    } else {
      const int i = u - n_qk;
      float v = lin_at(P, row, off_v + i);
      if (vmode == 1) vfirst[(long long)row * G * dv + i] = v;
      else if (vmode == 2) { const float lam = vmix[0]; v = (1.0f - lam) * v + lam * vfirst[(long long)row * G * dv + i]; }
      const int g = i / dv, d = i - g * dv;
      KT* vo = v_all ? v_pool + (page * m.page_tokens + in_page) * ((long long)G * dv) + i
                     : v_pool + ((page * G + g) * m.page_tokens + in_page) * dv + d;
      act_store<KT>(vo, v);
    }
  }
}

// The same for prompts in bf16 serving, eight neighbouring entries per thread (16-byte loads and stores): P is the bf16 matrix
// the tensor-core Linear left (no bias), queries leave as bf16 rows for the tensor-core attention.  Wants dk, dv, the row pitch
// and the column offsets to be multiples of 8, and the rotating part a multiple of 8 entries (pairs (2i, 2i+1)) or of 16
// (pairs (i, i + dims/2): a thread turns the 8 entries at d together with the 8 at d + dims/2).  grid (T), 256 threads.
__device__ __forceinline__ uint4 hy_pack8(const float* y) {
  return make_uint4(f2_to_bf2(y[0], y[1]), f2_to_bf2(y[2], y[3]), f2_to_bf2(y[4], y[5]), f2_to_bf2(y[6], y[7]));
}
__global__ void __launch_bounds__(256) hy_rope_append_vec_kernel(const bf16* __restrict__ P, long long ldp, int off_q, int off_k, int off_v, int H,
                                                                 int G, int dk, int dv, RotArgs r, bf16* __restrict__ q16,
                                                                 bf16* __restrict__ k_pool, bf16* __restrict__ v_pool, int v_all,
                                                                 const float* __restrict__ vmix, float* __restrict__ vfirst, int vmode,
                                                                 BatchMeta m) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int s = m.tok_seq[row], pos = m.tok_pos[row];
  const long long page = m.page_table[(long long)m.seq_slot[s] * m.max_pages + pos / m.page_tokens];
  const int in_page = pos % m.page_tokens;
  const int hp = r.dims >> 1, dk8 = dk >> 3;
  __shared__ float cs_tab[2 * HY_MAX_ROT_PAIRS];
  for (int j = threadIdx.x; j < hp; j += blockDim.x) hy_rot_cs(r, pos, j, &cs_tab[2 * j], &cs_tab[2 * j + 1]);
  __syncthreads();
  const bf16* prow = P + (long long)row * ldp;
  const int n_qk = (H + G) * dk8, total = n_qk + ((G * dv) >> 3);
  for (int u = threadIdx.x; u < total; u += blockDim.x) {
    if (u < n_qk) {
      const int hd = u / dk8, d = (u - hd * dk8) << 3;
      const bool is_q = hd < H;
      const int h = is_q ? hd : hd - H;
      const bf16* src = prow + (is_q ? off_q : off_k) + h * dk;
      bf16* dst = is_q ? q16 + (long long)row * H * dk + (long long)h * dk : k_pool + ((page * G + h) * m.page_tokens + in_page) * dk;
      float a[8], y0[8];
      if (d >= r.dims) {                       // entries that do not turn
        *reinterpret_cast<uint4*>(dst + d) = *reinterpret_cast<const uint4*>(src + d);
      } else if (!r.half) {                    // pairs (2i, 2i + 1): four of them in this chunk
        hy_load8(src + d, nullptr, a);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float c = cs_tab[2 * ((d >> 1) + i)], sn = cs_tab[2 * ((d >> 1) + i) + 1];
          y0[2 * i] = a[2 * i] * c - a[2 * i + 1] * sn;
          y0[2 * i + 1] = a[2 * i + 1] * c + a[2 * i] * sn;
        }
        *reinterpret_cast<uint4*>(dst + d) = hy_pack8(y0);
      } else if (d < hp) {                     // pairs (i, i + dims/2): this chunk and its partner
        float b[8], y1[8];
        hy_load8(src + d, nullptr, a);
        hy_load8(src + d + hp, nullptr, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float c = cs_tab[2 * (d + i)], sn = cs_tab[2 * (d + i) + 1];
          y0[i] = a[i] * c - b[i] * sn;
          y1[i] = b[i] * c + a[i] * sn;
        }
        *reinterpret_cast<uint4*>(dst + d) = hy_pack8(y0);
        *reinterpret_cast<uint4*>(dst + d + hp) = hy_pack8(y1);
      }                                        // chunks in [dims/2, dims) were written by their partners
    } else {
      const int i = (u - n_qk) << 3;
      float v[8];
      hy_load8(prow + off_v + i, nullptr, v);
      float* vf = vfirst + (long long)row * G * dv + i;
      if (vmode == 1) {
        *reinterpret_cast<float4*>(vf) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(vf + 4) = make_float4(v[4], v[5], v[6], v[7]);
      } else if (vmode == 2) {
        const float lam = vmix[0];
        const float4 f0 = *reinterpret_cast<const float4*>(vf), f1 = *reinterpret_cast<const float4*>(vf + 4);
        const float fv[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (1.0f - lam) * v[j] + lam * fv[j];
      }
      const int g = i / dv, d = i - g * dv;
      bf16* vo = v_all ? v_pool + (page * m.page_tokens + in_page) * ((long long)G * dv) + i
                       : v_pool + ((page * G + g) * m.page_tokens + in_page) * dv + d;
      *reinterpret_cast<uint4*>(vo) = hy_pack8(v);
    }
  }
}

// What follows the attention of an XB_MIX_SOFTMAX layer with mixed heads and / or head gates.
// talk != nullptr: o holds, per token and query head g, that head's softmax weights applied to the values of EVERY key head
// ([T][H][G * dv]); mixing the weights, w'_h = sum_g talk[h, g] w_g, and applying them to the values of head h's own key
// head c(h) is the same as  out_h = sum_g talk[h, g] o[g][c(h)]  (both are linear in the weights).  Else o is [T][H][dv].
// off_gate >= 0: head h is multiplied by sigmoid(P[t, off_gate + h]).  grid (T, ceil(H * dv / 256)).
template <typename AT, typename OT>
__global__ void __launch_bounds__(256) hy_heads_mix_kernel(const OT* __restrict__ o, const float* __restrict__ talk, LinOut P, int off_gate,
                                                           int H, int G, int dv, AT* __restrict__ out, long long ld_out) {
  pdl_launch_dependents();
  pdl_wait();
  const long long t = blockIdx.x;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= H * dv) return;
  const int h = i / dv, d = i - h * dv;
  float v;
  if (talk != nullptr) {
    const int c = h / (H / G);
    const OT* ot = o + t * ((long long)H * G * dv) + (long long)c * dv + d;
    v = 0.f;
    for (int g = 0; g < H; ++g) v = fmaf(talk[h * H + g], act_load<OT>(ot + (long long)g * G * dv), v);
  } else {
    v = act_load<OT>(o + t * ((long long)H * dv) + i);
  }
  if (off_gate >= 0) v *= hy_sigmoid(lin_at(P, t, off_gate + h));
  act_store<AT>(out + t * ld_out + i, v);
}

// The same on the bf16 matrix the tensor-core attention leaves, eight neighbouring channels per thread (dv a multiple of 8).
// grid (T, ceil(H * dv / 8 / 256)).
template <typename AT>
__global__ void __launch_bounds__(256) hy_heads_mix_vec_kernel(const bf16* __restrict__ o, const float* __restrict__ talk, LinOut P, int off_gate,
                                                               int H, int G, int dv, AT* __restrict__ out, long long ld_out) {
  pdl_launch_dependents();
  pdl_wait();
  const long long t = blockIdx.x;
  const int i8 = blockIdx.y * blockDim.x + threadIdx.x, dv8 = dv >> 3;
  if (i8 >= H * dv8) return;
  const int h = i8 / dv8, d = (i8 - h * dv8) << 3;
  float acc[8];
  if (talk != nullptr) {
    const int c = h / (H / G);
    const bf16* ot = o + t * ((long long)H * G * dv) + (long long)c * dv + d;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int g = 0; g < H; ++g) {
      float x[8];
      hy_load8(ot + (long long)g * G * dv, nullptr, x);
      const float w = talk[h * H + g];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(w, x[j], acc[j]);
    }
  } else {
    hy_load8(o + t * ((long long)H * dv) + (long long)h * dv + d, nullptr, acc);
  }
  if (off_gate >= 0) {
    const float gt = hy_sigmoid(lin_at(P, t, off_gate + h));
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= gt;
  }
  AT* dst = out + t * ld_out + (long long)h * dv + d;
#pragma unroll
  for (int j = 0; j < 8; ++j) act_store<AT>(dst + j, acc[j]);
}

// ----------------------------------------------------------------------------- feed-forward activation, side input, logits
template <typename AT>
__global__ void hy_relu2_kernel(LinOut u, AT* __restrict__ out, long long ld_out, int T, int F) {
  pdl_launch_dependents();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * F) return;
  const long long t = idx / F;
  const int i = (int)(idx - t * F);
  const float v = fmaxf(lin_at(u, t, i), 0.f);
  act_store<AT>(out + t * ld_out + i, v * v);
}

// the same on a bf16 matrix without bias, eight neighbours per thread (F, ld and ld_out multiples of 8)
__global__ void hy_relu2_vec_kernel(const bf16* __restrict__ u, long long ld, bf16* __restrict__ out, long long ld_out, int T, int F) {
  pdl_launch_dependents();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int f8 = F >> 3;
  if (idx >= (long long)T * f8) return;
  const long long t = idx / f8;
  const int i = (int)(idx - t * f8) << 3;
  const uint4 v = *reinterpret_cast<const uint4*>(u + t * ld + i);
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t r[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 f = bf2_to_f2(w[j]);
    f.x = fmaxf(f.x, 0.f); f.y = fmaxf(f.y, 0.f);
    r[j] = f2_to_bf2(f.x * f.x, f.y * f.y);
  }
  *reinterpret_cast<uint4*>(out + t * ld_out + i) = make_uint4(r[0], r[1], r[2], r[3]);
}

// g[t, i] = gelu_tanh(gate[t, i]) * side_embed[token[t], col0 + i]
template <typename AT>
__global__ void hy_side_gate_kernel(LinOut gate, const int* __restrict__ tokens, const bf16* __restrict__ side_embed, long long ld_se,
                                    int col0, int V, AT* __restrict__ out, long long ld_out, int T, int sd) {
  pdl_launch_dependents();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * sd) return;
  const long long t = idx / sd;
  const int i = (int)(idx - t * sd);
  int tok = tokens[t];
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
  act_store<AT>(out + t * ld_out + i, hy_gelu_tanh(lin_at(gate, t, i)) * bf2f(side_embed[(long long)tok * ld_se + col0 + i]));
}

// The whole per-layer token input for a few rows (decode steps), one block per row:
//   g = gelu_tanh(W_gate xa) * side_embed[token, col0 ..];  y = W_proj g;  x += y / rms(y) * side_norm;  hn = norm(x) * (1 + nw)
// with xa = x and g rounded to the activation type AT, as the separate Linears see them.  Dynamic smem (2 D + sd) floats.
template <typename AT>
__device__ __forceinline__ float act_round(float v);
template <> __device__ __forceinline__ float act_round<float>(float v) { return v; }
template <> __device__ __forceinline__ float act_round<bf16>(float v) { return bf2f(f2bf(v)); }
template <typename AT>
__global__ void __launch_bounds__(1024) hy_side_fused_kernel(float* __restrict__ x, const int* __restrict__ tokens, const bf16* __restrict__ side_embed,
                                                             long long ld_se, int col0, int V, const bf16* __restrict__ w_gate,
                                                             const bf16* __restrict__ w_proj, const float* __restrict__ side_norm,
                                                             const float* __restrict__ nw, float* __restrict__ hn, float eps, int D, int sd) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float sm[];
  __shared__ float red[32];
  float* g = sm;                        // sd floats, rounded up to a multiple of 4 (16-byte reads)
  float* xs = sm + ((sd + 3) & ~3);
  float* ys = xs + ((D + 3) & ~3);
  const long long t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  float* xr = x + t * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) xs[i] = act_round<AT>(xr[i]);
  __syncthreads();
  int tok = tokens[t];
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
  for (int i = warp; i < sd; i += nwarps) {
    const bf16* wr = w_gate + (long long)i * D;
    float d = 0.f;
    if ((D & 7) == 0) {
      for (int k = lane * 8; k < D; k += 256) d = hy_dot8(xs + k, *reinterpret_cast<const uint4*>(wr + k), d);
    } else {
      for (int k = lane; k < D; k += 32) d = fmaf(bf2f(wr[k]), xs[k], d);
    }
    d = warp_sum(d);
    if (lane == 0) g[i] = act_round<AT>(hy_gelu_tanh(d) * bf2f(side_embed[(long long)tok * ld_se + col0 + i]));
  }
  __syncthreads();
  float ss = 0.f;
  for (int j = threadIdx.x; j < D; j += blockDim.x) {
    const bf16* wr = w_proj + (long long)j * sd;
    float y = 0.f;
    if ((sd & 7) == 0) {
      for (int i = 0; i < sd; i += 8) y = hy_dot8(g + i, *reinterpret_cast<const uint4*>(wr + i), y);
    } else {
      for (int i = 0; i < sd; ++i) y = fmaf(bf2f(wr[i]), g[i], y);
    }
    ys[j] = y;
    ss += y * y;
  }
  ss = block_sum<1024>(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)D + eps);
  float s2 = 0.f;
  for (int j = threadIdx.x; j < D; j += blockDim.x) {
    const float v = xr[j] + ys[j] * inv * side_norm[j];
    xr[j] = v;
    ys[j] = v;
    s2 += v * v;
  }
  if (nw == nullptr) return;
  s2 = block_sum<1024>(s2, red);
  const float inv2 = 1.0f / sqrtf(s2 / (float)D + eps);
  for (int j = threadIdx.x; j < D; j += blockDim.x) hn[t * D + j] = ys[j] * inv2 * (1.0f + nw[j]);
}

// rows idx[r] of the normed stream as the head's input
template <typename AT>
__global__ void hy_gather_rows_kernel(const float* __restrict__ src, const int* __restrict__ idx, AT* __restrict__ dst, int D) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const float* s = src + (long long)idx[r] * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) act_store<AT>(dst + (long long)r * D + i, s[i]);
}

// logits <- cap * tanh(logits / cap) (cap > 0), from any Linear output into a dense fp32 [n, V]
__global__ void hy_logits_kernel(LinOut y, float cap, float* __restrict__ out, int n, int V) {
  pdl_launch_dependents();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n * V) return;
  const long long t = idx / V;
  const int i = (int)(idx - t * V);
  const float v = lin_at(y, t, i);
  out[idx] = cap > 0.f ? cap * tanhf(v / cap) : v;
}

// ----------------------------------------------------------------------------- latent attention
// Per token the fused projection P carries q (H heads of [dn unrotated | dr rotated]) and the down-projection
// [R latent | dr rotated key part].  One block per token:
//   cache row  = [ latent / rms(latent) * nw  |  rot(key part) ]      -> k_pool (one "key head", row of R + dr elements)
//   qa[t, h]   = [ (filled by hy_head_mm_t_kernel)  |  rot(q rotated part of head h) ]   fp32, rows of H * (R + dr)
// rot: entries 2i, 2i+1 (i < rot_dims / 2) turn by the angle pos * freq[i]; the others pass.  Angles are fp32.
template <typename KT>
__global__ void __launch_bounds__(256) hy_latent_prep_kernel(LinOut P, int off_q, int off_dkv, int H, int dn, int dr, int R, int rot_dims,
                                                             const float* __restrict__ freq, const float* __restrict__ nw, float eps,
                                                             KT* __restrict__ k_pool, BatchMeta m, float* __restrict__ qa) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  const int row = blockIdx.x;
  const int s = m.tok_seq[row], pos = m.tok_pos[row];
  const int page = m.page_table[(long long)m.seq_slot[s] * m.max_pages + pos / m.page_tokens];
  KT* kr = k_pool + ((long long)page * m.page_tokens + pos % m.page_tokens) * (R + dr);
  float ss = 0.f;
  for (int i = threadIdx.x; i < R; i += 256) {
    const float v = lin_at(P, row, off_dkv + i);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum<256>(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)R + eps);
  for (int i = threadIdx.x; i < R; i += 256) act_store<KT>(kr + i, lin_at(P, row, off_dkv + i) * inv * nw[i]);
  const int half = rot_dims >> 1, hp = dr - half;   // per vector: `half` pairs, then the entries that pass unchanged
  // vector 0 = the shared key part, 1 + h = head h's rotated query part
  for (int idx = threadIdx.x; idx < (H + 1) * hp; idx += 256) {
    const int vec = idx / hp, i = idx - vec * hp;
    const int src = vec == 0 ? off_dkv + R : off_q + (vec - 1) * (dn + dr) + dn;
    float* qd = qa + (long long)row * H * (R + dr) + (long long)(vec - 1) * (R + dr) + R;
    if (i < half) {
      const float u = lin_at(P, row, src + 2 * i), v = lin_at(P, row, src + 2 * i + 1);
      float sn, cs;
      sincosf((float)pos * freq[i], &sn, &cs);
      const float a = u * cs - v * sn, b = v * cs + u * sn;
      if (vec == 0) { act_store<KT>(kr + R + 2 * i, a); act_store<KT>(kr + R + 2 * i + 1, b); }
      else { qd[2 * i] = a; qd[2 * i + 1] = b; }
    } else {
      const int j = rot_dims + (i - half);
      const float v = lin_at(P, row, src + j);
      if (vec == 0) act_store<KT>(kr + R + j, v);
      else qd[j] = v;
    }
  }
}

// Per-head products with a weight that is stored head by head.
// "t" form (a query folded into the latent space): y[t, h * ldy + n] = sum_k X[t, xoff + h * xs + k] * W[(h * K + k) * N + n]
// grid (ceil(T / 8), H), 256 threads over n; the 8 rows' inputs sit in shared memory (8 * K floats).
#define HY_MM_ROWS 8
__global__ void __launch_bounds__(256) hy_head_mm_t_kernel(LinOut X, int xoff, int xs, const bf16* __restrict__ W, float* __restrict__ y,
                                                           long long ldy_row, int ldy, int T, int K, int N) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float xsm[];
  const int t0 = blockIdx.x * HY_MM_ROWS, h = blockIdx.y;
  const int nt = T - t0 < HY_MM_ROWS ? T - t0 : HY_MM_ROWS;
  for (int i = threadIdx.x; i < HY_MM_ROWS * K; i += 256) {
    const int r = i / K, k = i - r * K;
    xsm[i] = r < nt ? lin_at(X, t0 + r, xoff + h * xs + k) : 0.f;
  }
  __syncthreads();
  const bf16* Wh = W + (long long)h * K * N;
  for (int n = threadIdx.x; n < N; n += 256) {
    float acc[HY_MM_ROWS];
#pragma unroll
    for (int r = 0; r < HY_MM_ROWS; ++r) acc[r] = 0.f;
    for (int k = 0; k < K; ++k) {
      const float w = bf2f(Wh[(long long)k * N + n]);
#pragma unroll
      for (int r = 0; r < HY_MM_ROWS; ++r) acc[r] = fmaf(xsm[r * K + k], w, acc[r]);
    }
    for (int r = 0; r < nt; ++r) y[(long long)(t0 + r) * ldy_row + (long long)h * ldy + n] = acc[r];
  }
}
// plain form (a latent read-out turned into the head's value): y[t, h * N + n] = sum_k x[t, h * K + k] * W[(h * N + n) * K + k]
// grid (ceil(T / 8), H), 128 threads: a thread owns an output n and walks its weight row 16 bytes at a time against the 8 rows'
// inputs in shared memory (broadcast reads, no shuffles).
template <typename AT>
__global__ void __launch_bounds__(128) hy_head_mm_kernel(const float* __restrict__ x, long long ldx, const bf16* __restrict__ W,
                                                         AT* __restrict__ y, long long ldy, int T, int K, int N) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float xsm[];
  const int t0 = blockIdx.x * HY_MM_ROWS, h = blockIdx.y;
  const int nt = T - t0 < HY_MM_ROWS ? T - t0 : HY_MM_ROWS;
  for (int i = threadIdx.x; i < HY_MM_ROWS * K; i += 128) {
    const int r = i / K, k = i - r * K;
    xsm[i] = r < nt ? x[(long long)(t0 + r) * ldx + (long long)h * K + k] : 0.f;
  }
  __syncthreads();
  const bool vec = (K & 7) == 0 && (reinterpret_cast<uintptr_t>(W) & 15) == 0;
  for (int n = threadIdx.x; n < N; n += 128) {
    const bf16* wr = W + ((long long)h * N + n) * K;
    float acc[HY_MM_ROWS];
#pragma unroll
    for (int r = 0; r < HY_MM_ROWS; ++r) acc[r] = 0.f;
    if (vec) {
      for (int k = 0; k < K; k += 8) {
        const uint4 u = *reinterpret_cast<const uint4*>(wr + k);
        const float2 w0 = bf2_to_f2(u.x), w1 = bf2_to_f2(u.y), w2 = bf2_to_f2(u.z), w3 = bf2_to_f2(u.w);
#pragma unroll
        for (int r = 0; r < HY_MM_ROWS; ++r) {
          const float4 a = *reinterpret_cast<const float4*>(xsm + r * K + k), b = *reinterpret_cast<const float4*>(xsm + r * K + k + 4);
          float s = acc[r];
          s = fmaf(a.x, w0.x, s); s = fmaf(a.y, w0.y, s); s = fmaf(a.z, w1.x, s); s = fmaf(a.w, w1.y, s);
          s = fmaf(b.x, w2.x, s); s = fmaf(b.y, w2.y, s); s = fmaf(b.z, w3.x, s); s = fmaf(b.w, w3.y, s);
          acc[r] = s;
        }
      }
    } else {
      for (int k = 0; k < K; ++k) {
        const float w = bf2f(wr[k]);
#pragma unroll
        for (int r = 0; r < HY_MM_ROWS; ++r) acc[r] = fmaf(xsm[r * K + k], w, acc[r]);
      }
    }
    for (int r = 0; r < nt; ++r) act_store<AT>(y + (long long)(t0 + r) * ldy + (long long)h * N + n, acc[r]);
  }
}

// The read-out of all heads normed as ONE vector (RMS over the n entries of a token), weighted and gated by sigmoid:
// out[t, i] = o[t, i] / rms(o[t, :]) * w[i] * sigmoid(P[t, off_gate + i]).  grid (T), 256 threads.
template <typename AT>
__global__ void __launch_bounds__(256) hy_all_heads_norm_kernel(const float* __restrict__ o, long long ldo, const float* __restrict__ w, LinOut P,
                                                                int off_gate, float eps, AT* __restrict__ out, long long ld_out, int n) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  const long long t = blockIdx.x;
  const float* p = o + t * ldo;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += 256) ss = fmaf(p[i], p[i], ss);
  ss = block_sum<256>(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += 256) act_store<AT>(out + t * ld_out + i, p[i] * inv * w[i] * hy_sigmoid(lin_at(P, t, off_gate + i)));
}

// ----------------------------------------------------------------------------- element-wise activations of projection columns
// out[t, i] = act(P[t, off + i]), i < n.  act: 0 SiLU, 1 tanh.  grid (T, ceil(n / 256)).
template <typename OT>
__global__ void hy_act_cols_kernel(LinOut P, int off, int n, int act, OT* __restrict__ out, long long ld_out) {
  pdl_launch_dependents();
  pdl_wait();
  const long long t = blockIdx.x;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float z = lin_at(P, t, off + i);
  act_store<OT>(out + t * ld_out + i, act == 0 ? hy_silu(z) : tanhf(z));
}

// ----------------------------------------------------------------------------- general delta rule: what the recurrence reads
// From the fused projection P (r | k | v | gate | a | first decay projection) and the decay's second projection Wd, per
// token and head (n = key size = value size), all fp32:
//   w = exp(-e^-1/2 * sigmoid(Wd + w0)),  a = sigmoid(P_a)  (its bias comes with P),  u = k / sqrt(sum k^2 + 1e-6)
//   c row = [ r * w | u | w | a * u | k | v ] (six blocks of H * n),  ra = r . (a * u),  rk = r . k
// grid (T, ceil(H / 8)), a warp per head.
__global__ void __launch_bounds__(256) hy_gdelta_prep_kernel(LinOut P, int off_r, int off_k, int off_v, int off_a, LinOut Wd,
                                                             const float* __restrict__ w0, float* __restrict__ c, long long ldc,
                                                             float* __restrict__ ra, float* __restrict__ rk, int H, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const long long t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const long long HN = (long long)H * n;
  float* row = c + t * ldc;
  for (int h = blockIdx.y * nw + warp; h < H; h += nw * gridDim.y) {
    const int b = h * n;
    float sk = 0.f;
    for (int i = lane; i < n; i += 32) {
      const float k = lin_at(P, t, off_k + b + i);
      sk = fmaf(k, k, sk);
    }
    sk = warp_sum(sk);
    const float ik = 1.0f / sqrtf(sk + 1e-6f);
    float s_ra = 0.f, s_rk = 0.f;
    for (int i = lane; i < n; i += 32) {
      const float r = lin_at(P, t, off_r + b + i), k = lin_at(P, t, off_k + b + i);
      const float w = expf(-0.6065306597126334f * hy_sigmoid(lin_at(Wd, t, b + i) + w0[b + i]));
      const float a = hy_sigmoid(lin_at(P, t, off_a + b + i));
      const float u = k * ik, au = a * u;
      row[b + i] = r * w;
      row[HN + b + i] = u;
      row[2 * HN + b + i] = w;
      row[3 * HN + b + i] = au;
      row[4 * HN + b + i] = k;
      row[5 * HN + b + i] = lin_at(P, t, off_v + b + i);
      s_ra = fmaf(r, au, s_ra);
      s_rk = fmaf(r, k, s_rk);
    }
    s_ra = warp_sum(s_ra);
    s_rk = warp_sum(s_rk);
    if (lane == 0) { ra[t * H + h] = s_ra; rk[t * H + h] = s_rk; }
  }
}

// ----------------------------------------------------------------------------- clamped gated feed-forward, experts
__device__ __forceinline__ float hy_glu_clamp(float g, float u, float limit) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * hy_sigmoid(1.702f * g) * (u + 1.0f);
}
// One channel of one expert with routing weight w.  act: XB_ACT_GLU_CLAMP or XB_ACT_SWIGLU (silu(g) u, no limits).
// on_input: the weight multiplies what the expert reads, and since both projections are linear, (w h) W^T = w (h W^T):
// gate and up are scaled before the activation; otherwise the weight multiplies the activation (and so the output).
__device__ __forceinline__ float hy_expert_act(float g, float u, float w, float limit, int act, int on_input) {
  if (on_input) { g *= w; u *= w; }
  const float y = act == XB_ACT_SWIGLU ? hy_silu(g) * u : hy_glu_clamp(g, u, limit);
  return on_input ? y : w * y;
}
// U carries [gate (F) | up (F)] (biases on read): out[t, i] = glu(gate_i, up_i).  grid over T * F.
template <typename AT>
__global__ void hy_glu_clamp_kernel(LinOut U, int F, float limit, AT* __restrict__ out, long long ld_out, int T) {
  pdl_launch_dependents();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * F) return;
  const long long t = idx / F;
  const int i = (int)(idx - t * F);
  act_store<AT>(out + t * ld_out + i, hy_glu_clamp(lin_at(U, t, i), lin_at(U, t, F + i), limit));
}

// The same two activations on a bf16 matrix (prompts: the tcgen05 Linear's output), eight neighbours per thread.
// F, ld, ld_out and the column offsets are multiples of 8; bias (fp32, added first) may be nullptr.
__device__ __forceinline__ void hy_load8(const bf16* p, const float* bias, float* v) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const float2 a = bf2_to_f2(u.x), b = bf2_to_f2(u.y), c = bf2_to_f2(u.z), d = bf2_to_f2(u.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  if (bias != nullptr) {
    const float4 b0 = *reinterpret_cast<const float4*>(bias), b1 = *reinterpret_cast<const float4*>(bias + 4);
    v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w; v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
  }
}
__device__ __forceinline__ uint4 hy_glu8(const float* g, const float* u, float limit, float w, int act = XB_ACT_GLU_CLAMP, int on_input = 0) {
  float y[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) y[j] = hy_expert_act(g[j], u[j], w, limit, act, on_input);
  return make_uint4(f2_to_bf2(y[0], y[1]), f2_to_bf2(y[2], y[3]), f2_to_bf2(y[4], y[5]), f2_to_bf2(y[6], y[7]));
}
__global__ void hy_glu_clamp_vec_kernel(const bf16* __restrict__ u, long long ld, const float* __restrict__ bias, int F, float limit,
                                        bf16* __restrict__ out, long long ld_out, int T) {
  pdl_launch_dependents();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int f8 = F >> 3;
  if (idx >= (long long)T * f8) return;
  const long long t = idx / f8;
  const int i = (int)(idx - t * f8) << 3;
  float g[8], v[8];
  hy_load8(u + t * ld + i, bias != nullptr ? bias + i : nullptr, g);
  hy_load8(u + t * ld + F + i, bias != nullptr ? bias + F + i : nullptr, v);
  *reinterpret_cast<uint4*>(out + t * ld_out + i) = hy_glu8(g, v, limit, 1.0f);
}
__global__ void hy_moe_act_vec_kernel(const bf16* __restrict__ u, long long ld, const float* __restrict__ gw, int E, int f, float limit, int sf,
                                      float limit_s, int act, int on_input, bf16* __restrict__ out, long long ld_out, int T) {
  pdl_launch_dependents();
  pdl_wait();
  const int W8 = (E * f + sf) >> 3;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * W8) return;
  const long long t = idx / W8;
  const int i = (int)(idx - t * W8) << 3;
  float g[8], v[8];
  uint4 r = make_uint4(0u, 0u, 0u, 0u);
  if (i < E * f) {
    const int e = i / f, j = i - e * f;
    const float w = gw[t * E + e];
    if (w != 0.f) {
      hy_load8(u + t * ld + 2 * e * f + j, nullptr, g);
      hy_load8(u + t * ld + 2 * e * f + f + j, nullptr, v);
      r = hy_glu8(g, v, limit, w, act, on_input);
    }
  } else {
    const int j = i - E * f;
    hy_load8(u + t * ld + 2 * E * f + j, nullptr, g);
    hy_load8(u + t * ld + 2 * E * f + sf + j, nullptr, v);
    r = hy_glu8(g, v, limit_s, 1.0f, act, 0);
  }
  *reinterpret_cast<uint4*>(out + t * ld_out + i) = r;
}

// Router logits in fp32 for any number of rows: z[t, e] = sum_k x[t, k] w[e, k].  A warp takes one token and up to eight
// experts: it reads the token's row once and streams eight weight rows (which stay in L1 / L2 across tokens).
// grid (ceil(T * ceil(E / 8) / 8)), 256 threads.
// EPW: experts per warp, 8 for prompts; 1 in steps of few rows, where T * E warps are what fills the GPU.
template <typename AT, int EPW>
__global__ void __launch_bounds__(256) hy_router_logits_kernel(const AT* __restrict__ x, long long ldx, const bf16* __restrict__ w,
                                                               float* __restrict__ z, int T, int E, int K) {
  pdl_launch_dependents();
  pdl_wait();
  const int chunks = (E + EPW - 1) / EPW;
  const long long wid = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)T * chunks) return;
  const long long t = wid / chunks;
  const int e0 = (int)(wid - t * chunks) * EPW;
  const int ne = E - e0 < EPW ? E - e0 : EPW;
  const AT* xr = x + t * ldx;
  float acc[EPW];
#pragma unroll
  for (int j = 0; j < EPW; ++j) acc[j] = 0.f;
  if ((K & 7) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
    for (int k = lane * 8; k < K; k += 256) {
      float xv[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) xv[i] = act_load<AT>(xr + k + i);
#pragma unroll
      for (int j = 0; j < EPW; ++j) {
        if (j < ne) {
          const uint4 u = *reinterpret_cast<const uint4*>(w + (long long)(e0 + j) * K + k);
          const float2 a = bf2_to_f2(u.x), b = bf2_to_f2(u.y), c = bf2_to_f2(u.z), d = bf2_to_f2(u.w);
          float s = acc[j];
          s = fmaf(xv[0], a.x, s); s = fmaf(xv[1], a.y, s); s = fmaf(xv[2], b.x, s); s = fmaf(xv[3], b.y, s);
          s = fmaf(xv[4], c.x, s); s = fmaf(xv[5], c.y, s); s = fmaf(xv[6], d.x, s); s = fmaf(xv[7], d.y, s);
          acc[j] = s;
        }
      }
    }
  } else {
    for (int k = lane; k < K; k += 32) {
      const float xv = act_load<AT>(xr + k);
#pragma unroll
      for (int j = 0; j < EPW; ++j)
        if (j < ne) acc[j] = fmaf(xv, bf2f(w[(long long)(e0 + j) * K + k]), acc[j]);
    }
  }
#pragma unroll
  for (int j = 0; j < EPW; ++j) {
    const float v = warp_sum(acc[j]);
    if (lane == 0 && j < ne) z[t * E + e0 + j] = v;
  }
}

// Router: logits z [T, E] (fp32) -> dense weights gw [T, E], zero for experts a token does not use.
// scores = sigmoid(z); with groups > 0 the experts form `groups` equal groups of neighbours, a group is worth the sum of its
// two best scores and only experts of the `keep` best groups are eligible; the `top` best eligible experts get
// score * scale (no renormalisation).  Ties go to the lower index.  One warp per token; shared memory 2 * E + groups floats
// per warp.
// score_mode: XB_ROUTE_SIGMOID, or XB_ROUTE_SOFTMAX = softmax of the logits over all experts.  group_mode: XB_GROUP_TOP2 as above,
// or XB_GROUP_MAX = a group is worth its best score.  renorm: the chosen experts' scores are divided by their sum (+ 1e-20)
// before the scale.
__device__ __forceinline__ void hy_route_token(const float* __restrict__ zrow, float* sc, float* el, float* gs, int E, int top, int groups, int keep,
                                               float scale, float* __restrict__ gwrow, int score_mode, int group_mode, int renorm) {
  const int lane = threadIdx.x & 31;
  if (score_mode == XB_ROUTE_SOFTMAX) {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) { const float v = zrow[e]; sc[e] = v; mx = fmaxf(mx, v); }
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) { const float v = expf(sc[e] - mx); sc[e] = v; sum += v; }
    sum = warp_sum(sum);
    for (int e = lane; e < E; e += 32) { const float v = sc[e] / sum; sc[e] = v; el[e] = v; }
  } else {
    for (int e = lane; e < E; e += 32) {
      const float v = hy_sigmoid(zrow[e]);
      sc[e] = v;
      el[e] = v;
    }
  }
  __syncwarp();
  if (groups > 0 && keep < groups) {
    const int per = E / groups;
    for (int g = lane; g < groups; g += 32) {
      float b1 = -1.f, b2 = -1.f;
      for (int i = 0; i < per; ++i) {
        const float v = sc[g * per + i];
        if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) b2 = v;
      }
      gs[g] = group_mode == XB_GROUP_MAX ? b1 : b1 + (per > 1 ? b2 : 0.f);
    }
    __syncwarp();
    // a group stays when fewer than `keep` groups beat it (a tie counts for the lower index)
    for (int g = lane; g < groups; g += 32) {
      int better = 0;
      for (int o = 0; o < groups; ++o) better += (gs[o] > gs[g] || (gs[o] == gs[g] && o < g)) ? 1 : 0;
      if (better >= keep)
        for (int i = 0; i < per; ++i) el[g * per + i] = -1.f;
    }
    __syncwarp();
  }
  for (int e = lane; e < E; e += 32) gwrow[e] = 0.f;
  float tot = 0.f;   // sum of the chosen scores (every lane follows the same picks)
  for (int r = 0; r < top; ++r) {
    float bv = -1.f;
    int bi = E;
    for (int e = lane; e < E; e += 32)
      if (el[e] > bv) { bv = el[e]; bi = e; }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (bi >= E || bv < 0.f) break;
    tot += bv;
    if (lane == 0) { gwrow[bi] = sc[bi] * scale; el[bi] = -1.f; }
    __syncwarp();
  }
  if (renorm) {
    const float inv = 1.0f / (tot + 1e-20f);
    __syncwarp();
    for (int e = lane; e < E; e += 32) gwrow[e] *= inv;   // the entries of experts that were not chosen are zero
  }
}
__global__ void __launch_bounds__(128) hy_route_kernel(const float* __restrict__ z, int E, int top, int groups, int keep, float scale,
                                                       float* __restrict__ gw, int T, int score_mode, int group_mode, int renorm) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float rsm[];
  const int warp = threadIdx.x >> 5;
  const long long t = (long long)blockIdx.x * 4 + warp;
  if (t >= T) return;
  float* sc = rsm + (size_t)warp * (2 * E + (groups > 0 ? groups : 1));
  hy_route_token(z + t * E, sc, sc + E, sc + 2 * E, E, top, groups, keep, scale, gw + t * E, score_mode, group_mode, renorm);
}
// Steps of few rows: logits and routing of a token in ONE block of eight warps.  Warp w forms the fp32 logits of experts
// w, w + 8, ... (16-byte weight loads, fp32 sums, the order of hy_router_logits_kernel<AT, 1>), then the first warp routes.
// Shared memory: 3 * E + groups floats.  grid (T), 256 threads.
template <typename AT>
__global__ void __launch_bounds__(256) hy_router_route_kernel(const AT* __restrict__ x, long long ldx, const bf16* __restrict__ w, int K, int E, int top,
                                                              int groups, int keep, float scale, float* __restrict__ gw, int score_mode, int group_mode,
                                                              int renorm) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float rsm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long t = blockIdx.x;
  const AT* xr = x + t * ldx;
  const bool vec = (K & 7) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0;
  for (int e = warp; e < E; e += 8) {
    const bf16* wr = w + (long long)e * K;
    float acc = 0.f;
    if (vec) {
      for (int k = lane * 8; k < K; k += 256) {
        float wv[8];
        hy_load8(wr + k, nullptr, wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc = fmaf(act_load<AT>(xr + k + i), wv[i], acc);
      }
    } else {
      for (int k = lane; k < K; k += 32) acc = fmaf(act_load<AT>(xr + k), bf2f(wr[k]), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) rsm[e] = acc;
  }
  __syncthreads();
  if (warp == 0) hy_route_token(rsm, rsm + E, rsm + 2 * E, rsm + 3 * E, E, top, groups, keep, scale, gw + t * E, score_mode, group_mode, renorm);
}

// U carries, expert after expert, [gate_e (f) | up_e (f)], then the shared expert's [gate (sf) | up (sf)].
// out[t, e * f + i] = hy_expert_act(gate, up, gw[t, e]) (zero for experts the token does not use),
// out[t, E * f + i] = glu of the shared expert (limit_s): the input of ONE down projection over all experts' columns.
template <typename AT>
__global__ void hy_moe_act_kernel(LinOut U, const float* __restrict__ gw, int E, int f, float limit, int sf, float limit_s,
                                  int act, int on_input, AT* __restrict__ out, long long ld_out, int T) {
  pdl_launch_dependents();
  pdl_wait();
  const int W = E * f + sf;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * W) return;
  const long long t = idx / W;
  const int i = (int)(idx - t * W);
  float v = 0.f;
  if (i < E * f) {
    const int e = i / f, j = i - e * f;
    const float g = gw[t * E + e];
    if (g != 0.f) v = hy_expert_act(lin_at(U, t, 2 * e * f + j), lin_at(U, t, 2 * e * f + f + j), g, limit, act, on_input);
  } else {
    const int j = i - E * f;
    v = hy_expert_act(lin_at(U, t, 2 * E * f + j), lin_at(U, t, 2 * E * f + sf + j), 1.0f, limit_s, act, 0);
  }
  act_store<AT>(out + t * ld_out + i, v);
}

// Experts without a gate projection (XB_ACT_GELU): U carries every expert's up rows [up_e (f)], then the shared expert's (sf).
// out[t, e * f + i] = gw[t, e] * gelu(up) (zero for experts the token does not use), out[t, E * f + i] = gelu(up) of the shared
// expert: the input of ONE down projection over all experts' columns.  gelu is the exact form, 0.5 z (1 + erf(z / sqrt 2)).
__device__ __forceinline__ float hy_gelu_erf(float z) { return 0.5f * z * (1.0f + erff(z * 0.70710678118654752f)); }
template <typename AT>
__global__ void hy_moe_act1_kernel(LinOut U, const float* __restrict__ gw, int E, int f, int sf, AT* __restrict__ out, long long ld_out, int T) {
  pdl_launch_dependents();
  pdl_wait();
  const int W = E * f + sf;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * W) return;
  const long long t = idx / W;
  const int i = (int)(idx - t * W);
  float v = 0.f;
  if (i < E * f) {
    const float g = gw[t * E + i / f];
    if (g != 0.f) v = g * hy_gelu_erf(lin_at(U, t, i));
  } else {
    v = hy_gelu_erf(lin_at(U, t, i));
  }
  act_store<AT>(out + t * ld_out + i, v);
}
// the same on a bf16 matrix (prompts), eight neighbours per thread: f, sf, ld, ld_out multiples of 8
__global__ void hy_moe_act1_vec_kernel(const bf16* __restrict__ u, long long ld, const float* __restrict__ gw, int E, int f, int sf,
                                       bf16* __restrict__ out, long long ld_out, int T) {
  pdl_launch_dependents();
  pdl_wait();
  const int W8 = (E * f + sf) >> 3;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * W8) return;
  const long long t = idx / W8;
  const int i = (int)(idx - t * W8) << 3;
  const float w = i < E * f ? gw[t * E + i / f] : 1.0f;
  uint4 r = make_uint4(0u, 0u, 0u, 0u);
  if (w != 0.f) {
    float v[8];
    hy_load8(u + t * ld + i, nullptr, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = w * hy_gelu_erf(v[j]);
    r = make_uint4(f2_to_bf2(v[0], v[1]), f2_to_bf2(v[2], v[3]), f2_to_bf2(v[4], v[5]), f2_to_bf2(v[6], v[7]));
  }
  *reinterpret_cast<uint4*>(out + t * ld_out + i) = r;
}

// Experts gathered: steps of so few rows that most experts have no token read only the rows of the chosen experts instead of
// running every expert as one wide Linear.  gw [T, E] holds the routing weights (zero = not chosen; exactly `top` are not).
// Up: a warp per (token, chosen expert j, channel r) forms the gate and the up product of that channel (16-byte weight loads,
// fp32 sums) and applies hy_expert_act; out[t, j * F + r].  Wants D and F multiples of 8.  grid ceil(T * top * F / 8), 256 threads.
__device__ __forceinline__ int hy_nth_chosen(const float* __restrict__ gwt, int E, int j) {
  int seen = 0;
  for (int e = 0; e < E; ++e)
    if (gwt[e] != 0.f && seen++ == j) return e;
  return -1;
}
template <typename AT>
__global__ void __launch_bounds__(256) hy_moe_gather_up_kernel(const AT* __restrict__ x, long long ldx, const bf16* __restrict__ w_up,
                                                               const float* __restrict__ gw, int E, int top, int F, int D, float limit,
                                                               int act, int on_input, AT* __restrict__ out, int T) {
  pdl_launch_dependents();
  pdl_wait();
  const long long wid = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)T * top * F) return;
  const int t = (int)(wid / ((long long)top * F));
  const int rem = (int)(wid - (long long)t * top * F);
  const int j = rem / F, r = rem - j * F;
  const int e = hy_nth_chosen(gw + (long long)t * E, E, j);
  float v = 0.f;
  if (e >= 0) {
    const bf16* wg = w_up + ((long long)2 * e * F + r) * D;
    const bf16* wu = wg + (long long)F * D;
    const AT* xr = x + (long long)t * ldx;
    float g = 0.f, u = 0.f;
    for (int k = lane * 8; k < D; k += 256) {
      float xv[8], a[8], b[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) xv[i] = act_load<AT>(xr + k + i);
      hy_load8(wg + k, nullptr, a);
      hy_load8(wu + k, nullptr, b);
#pragma unroll
      for (int i = 0; i < 8; ++i) { g = fmaf(xv[i], a[i], g); u = fmaf(xv[i], b[i], u); }
    }
    g = warp_sum(g);
    u = warp_sum(u);
    v = hy_expert_act(g, u, gw[(long long)t * E + e], limit, act, on_input);
  }
  if (lane == 0) act_store<AT>(out + (long long)t * top * F + rem, v);
}
// Down: a warp per (token, output channel d) sums over the chosen experts' column blocks of the one down matrix [D, E * F].
// y [T, D] fp32.  grid ceil(T * D / 8), 256 threads.
template <typename AT>
__global__ void __launch_bounds__(256) hy_moe_gather_down_kernel(const AT* __restrict__ a, const bf16* __restrict__ w_down,
                                                                 const float* __restrict__ gw, int E, int top, int F, int D,
                                                                 float* __restrict__ y, int T) {
  pdl_launch_dependents();
  pdl_wait();
  const long long wid = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)T * D) return;
  const int t = (int)(wid / D), d = (int)(wid - (long long)t * D);
  const float* gwt = gw + (long long)t * E;
  const bf16* wrow = w_down + (long long)d * E * F;
  float acc = 0.f;
  int j = 0;
  for (int e = 0; e < E && j < top; ++e) {
    if (gwt[e] == 0.f) continue;
    const AT* ar = a + (long long)t * top * F + (long long)j * F;
    for (int k = lane * 8; k < F; k += 256) {
      float w[8];
      hy_load8(wrow + (long long)e * F + k, nullptr, w);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc = fmaf(act_load<AT>(ar + k + i), w[i], acc);
    }
    ++j;
  }
  acc = warp_sum(acc);
  if (lane == 0) y[(long long)t * D + d] = acc;
}

// ----------------------------------------------------------------------------- loader: any supported source type -> fp32 / bf16, strided rows
// src element types: 0 bf16, 1 fp16, 2 fp32 (the loader's codes).  rows x cols, destination row pitch ld_dst.
__device__ __forceinline__ float hy_src_at(const void* src, long long i, int dt) {
  if (dt == 0) return bf2f(reinterpret_cast<const bf16*>(src)[i]);
  if (dt == 1) return __half2float(reinterpret_cast<const __half*>(src)[i]);
  return reinterpret_cast<const float*>(src)[i];
}
template <typename OT>
__global__ void hy_load_convert_kernel(const void* __restrict__ src, int dt, long long rows, long long cols, OT* __restrict__ dst,
                                       long long ld_dst) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * cols) return;
  const long long r = idx / cols, c = idx - r * cols;
  act_store<OT>(dst + r * ld_dst + c, hy_src_at(src, idx, dt));
}
