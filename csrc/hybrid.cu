// Kernels of the hybrid decoder graphs (Kepovik): several residual streams mixed by hyper-connections, a hashed
// token-pair embedding, sigmoid (softmax-free) attention with a linear distance bias inside fixed position blocks over
// the paged KV cache, and the generalized delta-rule recurrence with a per-sequence fp32 state.
//
// Everything the design wants in 32-bit stays in fp32 here: the residual streams, every norm, attention scores and
// weights, decays / removal rates / unit keys and the recurrent state.  AT is the type of what feeds a matrix product
// (bf16 when serving, float for the all-fp32 mode); projections arrive as fp32 GEMM outputs.
// This translation unit is compiled WITHOUT --use_fast_math (exact expf / division / sqrt).
#include "kernels.h"

#include <cuda_bf16.h>

namespace b2b {
namespace {

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float ldf(const T* p, size_t i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, size_t i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p, size_t i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void stf(T* p, size_t i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, size_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }

__device__ __forceinline__ float warp_sum_(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float block_sum_(float v, float* sh) {
  v = warp_sum_(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = (threadIdx.x < nw) ? sh[threadIdx.x] : 0.f;
  if (w == 0) {
    r = warp_sum_(r);
    if (l == 0) sh[0] = r;
  }
  __syncthreads();
  return sh[0];
}

// dot product of a shared-memory fp32 vector with a cache row, 128-bit loads when the row allows it
template <typename T> __device__ __forceinline__ float dot_row(const float* q, const T* k, int n, bool vec);
template <> __device__ __forceinline__ float dot_row<float>(const float* q, const float* k, int n, bool vec) {
  float acc = 0.f;
  if (vec) {
    const float4* k4 = reinterpret_cast<const float4*>(k);
    for (int d = 0; d < n / 4; ++d) {
      const float4 v = k4[d];
      acc += q[4 * d] * v.x + q[4 * d + 1] * v.y + q[4 * d + 2] * v.z + q[4 * d + 3] * v.w;
    }
  } else {
    for (int d = 0; d < n; ++d) acc += q[d] * k[d];
  }
  return acc;
}
template <> __device__ __forceinline__ float dot_row<bf16>(const float* q, const bf16* k, int n, bool vec) {
  float acc = 0.f;
  if (vec) {
    const uint4* k8 = reinterpret_cast<const uint4*>(k);
    for (int d = 0; d < n / 8; ++d) {
      const uint4 v = k8[d];
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(p[j]);
        acc += q[8 * d + 2 * j] * f.x + q[8 * d + 2 * j + 1] * f.y;
      }
    }
  } else {
    for (int d = 0; d < n; ++d) acc += q[d] * __bfloat162float(k[d]);
  }
  return acc;
}

// ------------------------------------------------------------------------------------------------ embedding
// streams[t, s, :] = table[id] + pair[(prev * mul_prev + id * mul_cur) % buckets]   (row `buckets` at position 0)
// for every stream s.  The previous token of a span's first token comes from the sequence state (prev_tok[slot]).
// grid (token chunks, sequences).
template <typename WT>
__global__ void hyb_embed_kernel(const int* __restrict__ ids, const int* __restrict__ positions,
                                 const int* __restrict__ q_start, const int* __restrict__ q_len,
                                 const int* __restrict__ seq_slot, const int* __restrict__ prev_tok,
                                 const WT* __restrict__ table, const WT* __restrict__ pair, int buckets,
                                 long long mul_prev, long long mul_cur, float* __restrict__ streams, int ns, int W,
                                 int vocab, int tpb) {
  const int s = blockIdx.y;
  const int n = q_len[s];
  const int i0 = blockIdx.x * tpb;
  if (i0 >= n) return;
  const int t0 = q_start[s];
  const int i1 = min(n, i0 + tpb);
  for (int i = i0; i < i1; ++i) {
    const int t = t0 + i;
    int id = ids[t];
    id = min(max(id, 0), vocab - 1);
    long long row = -1;
    if (pair != nullptr) {
      if (positions[t] == 0) {
        row = buckets;
      } else {
        const long long prev = (i == 0) ? prev_tok[seq_slot[s]] : ids[t - 1];
        row = (prev * mul_prev + static_cast<long long>(id) * mul_cur) % buckets;
        if (row < 0) row += buckets;
      }
    }
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      float v = ldf(table, static_cast<size_t>(id) * W + c);
      if (row >= 0) v += ldf(pair, static_cast<size_t>(row) * W + c);
      for (int k = 0; k < ns; ++k) streams[(static_cast<size_t>(t) * ns + k) * W + c] = v;
    }
  }
}

// last token of every span -> sequence state (runs after the embedding of the step has read the old value)
__global__ void hyb_commit_prev_kernel(const int* __restrict__ ids, const int* __restrict__ q_start,
                                       const int* __restrict__ q_len, const int* __restrict__ seq_slot,
                                       int* __restrict__ prev_tok, int n_seqs) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= n_seqs) return;
  const int n = q_len[s];
  if (n <= 0) return;
  prev_tok[seq_slot[s]] = ids[q_start[s] + n - 1];
}

// --------------------------------------------------------------------------------------- hyper-connections
// One block per token row.  Optional "post" of the sublayer that just ran (y != null):
//     x_j <- sum_k mix[k, j] x_k + mult * out[j] * y            (all streams from the old ones)
// then optional "pre" of the next sublayer (gamma != null):
//     u = sum_k in[k] x_k ;  h = u / sqrt(mean(u^2) + eps) * (1 + gamma)      -> AT, row `out_row` of h
// With one stream and mix = in = out = 1 this is the plain pre-norm residual.
constexpr int NS_MAX = 16;

template <typename OT>
__device__ __forceinline__ void hc_row(float* __restrict__ streams, int t, int out_row, const float* __restrict__ y,
                                       int ld_y, const float* mix, const float* outw, float mult, const float* inw,
                                       const float* __restrict__ gamma, float eps, OT* __restrict__ h, int ld_h, int ns,
                                       int W, int write_back, float* ubuf, float* red) {
  float ssq = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float x[NS_MAX];
#pragma unroll
    for (int k = 0; k < NS_MAX; ++k)
      if (k < ns) x[k] = streams[(static_cast<size_t>(t) * ns + k) * W + c];
    if (y != nullptr) {
      const float yv = y[static_cast<size_t>(t) * ld_y + c];
      float nx[NS_MAX];
#pragma unroll
      for (int j = 0; j < NS_MAX; ++j) {
        if (j < ns) {
          float a = 0.f;
#pragma unroll
          for (int k = 0; k < NS_MAX; ++k)
            if (k < ns) a += mix[k * ns + j] * x[k];
          nx[j] = a + (mult * outw[j]) * yv;
        }
      }
#pragma unroll
      for (int j = 0; j < NS_MAX; ++j) {
        if (j < ns) {
          x[j] = nx[j];
          if (write_back) streams[(static_cast<size_t>(t) * ns + j) * W + c] = nx[j];
        }
      }
    }
    if (gamma != nullptr) {
      float u = 0.f;
#pragma unroll
      for (int k = 0; k < NS_MAX; ++k)
        if (k < ns) u += inw[k] * x[k];
      ubuf[c] = u;
      ssq += u * u;
    }
  }
  if (gamma == nullptr) return;
  ssq = block_sum_(ssq, red);
  const float rinv = 1.f / sqrtf(ssq / static_cast<float>(W) + eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x)
    stf(h, static_cast<size_t>(out_row) * ld_h + c, ubuf[c] * rinv * (1.f + gamma[c]));
}

// rows given by (sequence, token-in-span): grid (token chunks, sequences)
template <typename OT>
__global__ void __launch_bounds__(256) hc_step_kernel(float* streams, const int* __restrict__ q_start, const int* __restrict__ q_len,
                               const int* __restrict__ rows, const float* y, int ld_y, const float* __restrict__ mix_g,
                               const float* __restrict__ outw_g, float mult, const float* __restrict__ inw_g,
                               const float* gamma, float eps, OT* h, int ld_h, int ns, int W, int tpb) {
  extern __shared__ float smem[];
  float* ubuf = smem;                       // [W]
  float* coef = smem + W;                   // mix [ns*ns], out [ns], in [ns]
  __shared__ float red[32];
  for (int i = threadIdx.x; i < ns * ns; i += blockDim.x) coef[i] = mix_g ? mix_g[i] : (i / ns == i % ns ? 1.f : 0.f);
  for (int i = threadIdx.x; i < ns; i += blockDim.x) {
    coef[ns * ns + i] = outw_g ? outw_g[i] : 1.f;
    coef[ns * ns + ns + i] = inw_g ? inw_g[i] : 1.f;
  }
  __syncthreads();
  const float* mix = coef;
  const float* outw = coef + ns * ns;
  const float* inw = outw + ns;
  if (rows != nullptr) {                    // gathered rows (logit rows): output row = blockIdx.x, nothing written back
    hc_row<OT>(streams, rows[blockIdx.x], blockIdx.x, y, ld_y, mix, outw, mult, inw, gamma, eps, h, ld_h, ns, W, 0, ubuf, red);
    return;
  }
  const int s = blockIdx.y;
  const int n = q_len[s];
  const int i0 = blockIdx.x * tpb;
  if (i0 >= n) return;
  const int t0 = q_start[s];
  const int i1 = min(n, i0 + tpb);
  for (int i = i0; i < i1; ++i) {
    hc_row<OT>(streams, t0 + i, t0 + i, y, ld_y, mix, outw, mult, inw, gamma, eps, h, ld_h, ns, W, 1, ubuf, red);
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------------ activations
// out[t, c] = act(in[t, off + c]) for c < n   (1 = tanh, 2 = squared relu, 0 = copy)
template <typename OT>
__global__ void act_cols_kernel(const float* __restrict__ in, int ld_in, int off, OT* __restrict__ out, int ld_out,
                                int n, int act, size_t total) {
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / n;
    const int c = static_cast<int>(i % n);
    float v = in[t * ld_in + off + c];
    if (act == 1) v = tanhf(v);
    else if (act == 2) { v = fmaxf(v, 0.f); v = v * v; }
    stf(out, t * ld_out + c, v);
  }
}

// ---------------------------------------------------------------------------- attention: norms + cache append
// proj [T, ld] fp32 = [q (H*D) | k (G*D) | v (G*V) | gate (H*V)].  One warp per (token, head unit):
// q / k heads get an RMS norm over D with a plain weight shared by all heads; k and v rows go to the paged cache.
template <typename CT>
__global__ void attn_prep_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ qn,
                                 const float* __restrict__ kn, const int* __restrict__ slots, float* __restrict__ q_out,
                                 CT* __restrict__ k_cache, CT* __restrict__ v_cache, int T, int H, int G, int D, int V,
                                 float eps) {
  const int units = H + 2 * G;
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= static_cast<long long>(T) * units) return;
  const int t = static_cast<int>(wid / units), u = static_cast<int>(wid % units);
  const float* row = proj + static_cast<size_t>(t) * ld;
  if (u < H + G) {
    const bool isq = u < H;
    const float* src = row + (isq ? u * D : H * D + (u - H) * D);
    const int slot = isq ? 0 : slots[t];
    if (!isq && slot < 0) return;
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) ss += src[d] * src[d];
    ss = warp_sum_(ss);
    const float r = 1.f / sqrtf(ss / static_cast<float>(D) + eps);
    const float* w = isq ? qn : kn;
    if (isq) {
      float* dst = q_out + (static_cast<size_t>(t) * H + u) * D;
      for (int d = lane; d < D; d += 32) dst[d] = src[d] * r * w[d];
    } else {
      CT* dst = k_cache + (static_cast<size_t>(slot) * G + (u - H)) * D;
      for (int d = lane; d < D; d += 32) stf(dst, d, src[d] * r * w[d]);
    }
  } else {
    const int g = u - H - G;
    const int slot = slots[t];
    if (slot < 0) return;
    const float* src = row + H * D + G * D + g * V;
    CT* dst = v_cache + (static_cast<size_t>(slot) * G + g) * V;
    for (int d = lane; d < V; d += 32) stf(dst, d, src[d]);
  }
}

// ------------------------------------------------------------------------------------- sigmoid attention
// out[t, h, :] = sigmoid(gate[t, h, :]) * sum_j sigmoid(q_t . k_j * scale - slope_h (i - j) + pb[h]) v_j
// over the keys j <= i of the same block of `chunk` positions (chunk = 0: every j <= i); no normalisation over keys.
// slope_h = 2^(-8 (h + 1) / H).  Positions count from the start of the sequence: i = kv_len - q_len + index in span.
// One warp per (query, head); a pass over 32 keys computes one score per lane, then the lanes own value channels.
// grid (query tiles of 4, heads, sequences), 128 threads, dynamic smem 4 * D floats.
constexpr int ATT_WARPS = 4;
constexpr int ATT_VR = 8;        // value channels per lane: V <= 256

template <typename CT, typename OT>
__global__ void sig_attention_kernel(const float* __restrict__ q, const CT* __restrict__ k_cache,
                                     const CT* __restrict__ v_cache, const float* __restrict__ gate, int ld_gate,
                                     int gate_off, const float* __restrict__ pb, OT* __restrict__ out, int ld_out,
                                     const int* __restrict__ block_table, int max_pages, const int* __restrict__ q_start,
                                     const int* __restrict__ q_len, const int* __restrict__ kv_len, int H, int G, int D,
                                     int V, int chunk, float scale) {
  extern __shared__ float qs_all[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int s = blockIdx.z, hd = blockIdx.y;
  const int i = blockIdx.x * ATT_WARPS + warp;
  const int n = q_len[s];
  if (i >= n) return;                                  // (no block-wide barrier below)
  const int t = q_start[s] + i;
  const int pi = kv_len[s] - n + i;
  const int lo = chunk > 0 ? (pi / chunk) * chunk : 0;
  const int g = hd / (H / G);
  float* qs = qs_all + warp * D;
  const float* qrow = q + (static_cast<size_t>(t) * H + hd) * D;
  for (int d = lane; d < D; d += 32) qs[d] = qrow[d] * scale;
  __syncwarp();
  const float slope = exp2f(-8.f * static_cast<float>(hd + 1) / static_cast<float>(H));
  const float bias = pb[hd];
  const int* bt = block_table + static_cast<size_t>(s) * max_pages;
  const bool kvec = (D * sizeof(CT)) % 16 == 0;
  float acc[ATT_VR];
#pragma unroll
  for (int r = 0; r < ATT_VR; ++r) acc[r] = 0.f;
  for (int j0 = lo; j0 <= pi; j0 += 32) {
    const int j = j0 + lane;
    float wgt = 0.f;
    long long slot = 0;
    if (j <= pi) {
      slot = static_cast<long long>(bt[j >> 6]) * 64 + (j & 63);
      const float dot = dot_row<CT>(qs, k_cache + (static_cast<size_t>(slot) * G + g) * D, D, kvec);
      wgt = sigmoidf_(dot - slope * static_cast<float>(pi - j) + bias);
    }
    const int cnt = min(32, pi - j0 + 1);
    for (int jj = 0; jj < cnt; ++jj) {
      const float w = __shfl_sync(0xffffffffu, wgt, jj);
      const long long sl = __shfl_sync(0xffffffffu, slot, jj);
      const CT* vrow = v_cache + (static_cast<size_t>(sl) * G + g) * V;
#pragma unroll
      for (int r = 0; r < ATT_VR; ++r) {
        const int d = lane + 32 * r;
        if (d < V) acc[r] += w * ldf(vrow, d);
      }
    }
  }
  const float* grow = gate + static_cast<size_t>(t) * ld_gate + gate_off + hd * V;
#pragma unroll
  for (int r = 0; r < ATT_VR; ++r) {
    const int d = lane + 32 * r;
    if (d < V) stf(out, static_cast<size_t>(t) * ld_out + hd * V + d, acc[r] * sigmoidf_(grow[d]));
  }
}

// ------------------------------------------------------------------------------ generalized delta rule
// Per head, state S [dk, dv] (fp32, one per sequence slot), per token with r, k, v in R^dk / R^dv:
//     w = exp(-e^(-1/2) sigmoid(lora + w0))            decay per key channel
//     a = sigmoid(a_proj + a_bias)                     removal rate per key channel
//     u = k / sqrt(sum k^2 + 1e-6)
//     S <- diag(w) S - (a * u) (u^T S) + k v^T         (both products read the old S)
//     o = S^T r
// Columns of S are independent: a block owns DV_B columns of one (sequence, head); 8 lanes share a column, each with
// R consecutive key channels in registers (dk padded to 8 R with zeros).  Tokens are staged TT at a time in shared
// memory where w, a, u are prepared in parallel; the scan itself is sequential in the tokens of the span.
// proj [T, ld] fp32 holds r | k | v | gate | a (offsets given); lora [T, ld_l] fp32.
constexpr int DL_LANES = 8;
constexpr int DL_COLS = 32;      // columns per block -> 256 threads

template <int R>
__global__ void __launch_bounds__(DL_LANES* DL_COLS)
    delta_scan_kernel(const float* __restrict__ proj, int ld, int off_r, int off_k, int off_v, int off_a,
                      const float* __restrict__ lora, int ld_l, const float* __restrict__ w0,
                      const float* __restrict__ a_bias, float* __restrict__ state, float* __restrict__ out, int ld_out,
                      const int* __restrict__ q_start, const int* __restrict__ q_len, const int* __restrict__ kv_len,
                      const int* __restrict__ seq_slot, int H, int dk, int dv, int TT) {
  constexpr int DKP = R * DL_LANES;
  extern __shared__ float sm[];
  float* rs = sm;                    // [TT][DKP]
  float* ks = rs + TT * DKP;
  float* ws = ks + TT * DKP;
  float* aus = ws + TT * DKP;
  float* us = aus + TT * DKP;
  float* vs = us + TT * DKP;         // [TT][DL_COLS]
  const int s = blockIdx.z, hd = blockIdx.y;
  const int n = q_len[s];
  if (n <= 0) return;
  const int t0 = q_start[s];
  const int pos0 = kv_len[s] - n;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int col = tid / DL_LANES, l = tid % DL_LANES;
  const int cg = blockIdx.x * DL_COLS + col;
  const bool cok = cg < dv;
  float* S_g = state + (static_cast<size_t>(seq_slot[s]) * H + hd) * static_cast<size_t>(dk) * dv;
  float S[R];
#pragma unroll
  for (int m = 0; m < R; ++m) {
    const int i = l * R + m;
    S[m] = (pos0 > 0 && cok && i < dk) ? S_g[static_cast<size_t>(i) * dv + cg] : 0.f;
  }
  const float decay_c = 0.60653065971263342f;      // e^(-1/2)
  for (int tb = 0; tb < n; tb += TT) {
    const int nt = min(TT, n - tb);
    __syncthreads();
    // ---- stage: one warp per token
    for (int tt = warp; tt < nt; tt += (DL_LANES * DL_COLS) / 32) {
      const size_t t = static_cast<size_t>(t0 + tb + tt);
      const float* prow = proj + t * ld + hd * dk;
      const float* lrow = lora + t * ld_l + hd * dk;
      float ss = 0.f;
      for (int i = lane; i < dk; i += 32) {
        const float kk = prow[off_k + i];
        ss += kk * kk;
      }
      ss = warp_sum_(ss);
      const float rinv = 1.f / sqrtf(ss + 1e-6f);
      for (int i = lane; i < DKP; i += 32) {
        float rv = 0.f, kv = 0.f, wv = 0.f, av = 0.f, uv = 0.f;
        if (i < dk) {
          rv = prow[off_r + i];
          kv = prow[off_k + i];
          wv = expf(-decay_c * sigmoidf_(lrow[i] + w0[hd * dk + i]));
          uv = kv * rinv;
          av = sigmoidf_(prow[off_a + i] + a_bias[hd * dk + i]) * uv;
        }
        rs[tt * DKP + i] = rv;
        ks[tt * DKP + i] = kv;
        ws[tt * DKP + i] = wv;
        aus[tt * DKP + i] = av;
        us[tt * DKP + i] = uv;
      }
      const float* vrow = proj + t * ld + off_v + hd * dv;
      {
        const int c = blockIdx.x * DL_COLS + lane;
        vs[tt * DL_COLS + lane] = c < dv ? vrow[c] : 0.f;
      }
    }
    __syncthreads();
    // ---- scan
    for (int tt = 0; tt < nt; ++tt) {
      const float* up = us + tt * DKP + l * R;
      const float* wp = ws + tt * DKP + l * R;
      const float* ap = aus + tt * DKP + l * R;
      const float* kp = ks + tt * DKP + l * R;
      const float* rp = rs + tt * DKP + l * R;
      const float vj = vs[tt * DL_COLS + col];
      float part = 0.f;
#pragma unroll
      for (int m = 0; m < R; ++m) part += up[m] * S[m];
      part += __shfl_xor_sync(0xffffffffu, part, 1);
      part += __shfl_xor_sync(0xffffffffu, part, 2);
      part += __shfl_xor_sync(0xffffffffu, part, 4);
      float o = 0.f;
#pragma unroll
      for (int m = 0; m < R; ++m) {
        S[m] = wp[m] * S[m] - ap[m] * part + kp[m] * vj;
        o += S[m] * rp[m];
      }
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      o += __shfl_xor_sync(0xffffffffu, o, 4);
      if (l == 0 && cok) out[static_cast<size_t>(t0 + tb + tt) * ld_out + hd * dv + cg] = o;
    }
  }
  if (cok) {
#pragma unroll
    for (int m = 0; m < R; ++m) {
      const int i = l * R + m;
      if (i < dk) S_g[static_cast<size_t>(i) * dv + cg] = S[m];
    }
  }
}

// o [T, H*dv] fp32 -> per head: o / sqrt(mean(o^2) + eps) * weight * sigmoid(gate)   -> AT.  One warp per (token, head).
template <typename OT>
__global__ void delta_post_kernel(const float* __restrict__ o, int ld_o, const float* __restrict__ gate, int ld_g,
                                  int off_g, const float* __restrict__ weight, OT* __restrict__ out, int ld_out, int T,
                                  int H, int dv, float eps) {
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= static_cast<long long>(T) * H) return;
  const int t = static_cast<int>(wid / H), hd = static_cast<int>(wid % H);
  const float* src = o + static_cast<size_t>(t) * ld_o + hd * dv;
  const float* grow = gate + static_cast<size_t>(t) * ld_g + off_g + hd * dv;
  float ss = 0.f;
  for (int d = lane; d < dv; d += 32) ss += src[d] * src[d];
  ss = warp_sum_(ss);
  const float r = 1.f / sqrtf(ss / static_cast<float>(dv) + eps);
  for (int d = lane; d < dv; d += 32)
    stf(out, static_cast<size_t>(t) * ld_out + hd * dv + d, src[d] * r * weight[hd * dv + d] * sigmoidf_(grow[d]));
}

inline int last_error() { return static_cast<int>(cudaGetLastError()); }

}  // namespace

// ================================================================================================ launchers
int launch_hyb_embed(const int* ids, const int* positions, const int* q_start, const int* q_len, const int* seq_slot,
                     const int* prev_tok, const void* table, const void* pair, int buckets, long long mul_prev,
                     long long mul_cur, float* streams, int ns, int W, int vocab, int n_seqs, int max_q, int f32,
                     cudaStream_t s) {
  if (n_seqs <= 0 || max_q <= 0) return 0;
  const int tpb = 4;
  dim3 grid((max_q + tpb - 1) / tpb, n_seqs);
  if (f32)
    hyb_embed_kernel<float><<<grid, 256, 0, s>>>(ids, positions, q_start, q_len, seq_slot, prev_tok,
                                                 static_cast<const float*>(table), static_cast<const float*>(pair),
                                                 buckets, mul_prev, mul_cur, streams, ns, W, vocab, tpb);
  else
    hyb_embed_kernel<bf16><<<grid, 256, 0, s>>>(ids, positions, q_start, q_len, seq_slot, prev_tok,
                                                static_cast<const bf16*>(table), static_cast<const bf16*>(pair), buckets,
                                                mul_prev, mul_cur, streams, ns, W, vocab, tpb);
  return last_error();
}

int launch_hyb_commit_prev(const int* ids, const int* q_start, const int* q_len, const int* seq_slot, int* prev_tok,
                           int n_seqs, cudaStream_t s) {
  if (n_seqs <= 0) return 0;
  hyb_commit_prev_kernel<<<(n_seqs + 127) / 128, 128, 0, s>>>(ids, q_start, q_len, seq_slot, prev_tok, n_seqs);
  return last_error();
}

int launch_hc_step(float* streams, const int* q_start, const int* q_len, const int* rows, int n_rows, int n_seqs,
                   int max_q, const float* y, int ld_y, const float* mix, const float* outw, float mult,
                   const float* inw, const float* gamma, float eps, void* h, int ld_h, int ns, int W, int f32,
                   cudaStream_t s) {
  if (ns < 1 || ns > NS_MAX) return -2;
  const int tpb = 2;
  dim3 grid;
  if (rows != nullptr) {
    if (n_rows <= 0) return 0;
    grid = dim3(n_rows);
  } else {
    if (n_seqs <= 0 || max_q <= 0) return 0;
    grid = dim3((max_q + tpb - 1) / tpb, n_seqs);
  }
  const size_t smem = (static_cast<size_t>(W) + ns * ns + 2 * ns) * sizeof(float);
  const int threads = 256;
  if (f32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(hc_step_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    hc_step_kernel<float><<<grid, threads, smem, s>>>(streams, q_start, q_len, rows, y, ld_y, mix, outw, mult, inw, gamma,
                                                      eps, static_cast<float*>(h), ld_h, ns, W, tpb);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(hc_step_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    hc_step_kernel<bf16><<<grid, threads, smem, s>>>(streams, q_start, q_len, rows, y, ld_y, mix, outw, mult, inw, gamma,
                                                     eps, static_cast<bf16*>(h), ld_h, ns, W, tpb);
  }
  return last_error();
}

int launch_act_cols(const float* in, int ld_in, int off, void* out, int ld_out, int n, int act, int T, int f32,
                    cudaStream_t s) {
  const size_t total = static_cast<size_t>(T) * n;
  if (total == 0) return 0;
  const int blocks = static_cast<int>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
  if (f32) act_cols_kernel<float><<<blocks, 256, 0, s>>>(in, ld_in, off, static_cast<float*>(out), ld_out, n, act, total);
  else act_cols_kernel<bf16><<<blocks, 256, 0, s>>>(in, ld_in, off, static_cast<bf16*>(out), ld_out, n, act, total);
  return last_error();
}

int launch_attn_prep(const float* proj, int ld, const float* qn, const float* kn, const int* slots, float* q_out,
                     void* k_cache, void* v_cache, int T, int H, int G, int D, int V, float eps, int f32,
                     cudaStream_t s) {
  const long long warps = static_cast<long long>(T) * (H + 2 * G);
  if (warps <= 0) return 0;
  const int blocks = static_cast<int>((warps + 3) / 4);
  if (f32)
    attn_prep_kernel<float><<<blocks, 128, 0, s>>>(proj, ld, qn, kn, slots, q_out, static_cast<float*>(k_cache),
                                                   static_cast<float*>(v_cache), T, H, G, D, V, eps);
  else
    attn_prep_kernel<bf16><<<blocks, 128, 0, s>>>(proj, ld, qn, kn, slots, q_out, static_cast<bf16*>(k_cache),
                                                  static_cast<bf16*>(v_cache), T, H, G, D, V, eps);
  return last_error();
}

int launch_sig_attention(const float* q, const void* k_cache, const void* v_cache, const float* gate, int ld_gate,
                         int gate_off, const float* pb, void* out, int ld_out, const int* block_table, int max_pages,
                         const int* q_start, const int* q_len, const int* kv_len, int n_seqs, int max_q, int H, int G,
                         int D, int V, int chunk, float scale, int f32, cudaStream_t s) {
  if (n_seqs <= 0 || max_q <= 0) return 0;
  if (V > 32 * ATT_VR || G <= 0 || H % G != 0) return -2;
  dim3 grid((max_q + ATT_WARPS - 1) / ATT_WARPS, H, n_seqs);
  const size_t smem = static_cast<size_t>(ATT_WARPS) * D * sizeof(float);
  if (f32)
    sig_attention_kernel<float, float><<<grid, 32 * ATT_WARPS, smem, s>>>(
        q, static_cast<const float*>(k_cache), static_cast<const float*>(v_cache), gate, ld_gate, gate_off, pb,
        static_cast<float*>(out), ld_out, block_table, max_pages, q_start, q_len, kv_len, H, G, D, V, chunk, scale);
  else
    sig_attention_kernel<bf16, bf16><<<grid, 32 * ATT_WARPS, smem, s>>>(
        q, static_cast<const bf16*>(k_cache), static_cast<const bf16*>(v_cache), gate, ld_gate, gate_off, pb,
        static_cast<bf16*>(out), ld_out, block_table, max_pages, q_start, q_len, kv_len, H, G, D, V, chunk, scale);
  return last_error();
}

template <int R>
static int launch_delta_r(const float* proj, int ld, int off_r, int off_k, int off_v, int off_a, const float* lora,
                          int ld_l, const float* w0, const float* a_bias, float* state, float* out, int ld_out,
                          const int* q_start, const int* q_len, const int* kv_len, const int* seq_slot, int n_seqs, int H,
                          int dk, int dv, cudaStream_t s) {
  constexpr int DKP = R * DL_LANES;
  const int TT = DKP <= 64 ? 16 : (DKP == 128 ? 8 : 4);
  const size_t smem = static_cast<size_t>(TT) * (5 * DKP + DL_COLS) * sizeof(float);
  dim3 grid((dv + DL_COLS - 1) / DL_COLS, H, n_seqs);
  delta_scan_kernel<R><<<grid, DL_LANES * DL_COLS, smem, s>>>(proj, ld, off_r, off_k, off_v, off_a, lora, ld_l, w0, a_bias,
                                                              state, out, ld_out, q_start, q_len, kv_len, seq_slot, H, dk,
                                                              dv, TT);
  return last_error();
}

int launch_delta_scan(const float* proj, int ld, int off_r, int off_k, int off_v, int off_a, const float* lora, int ld_l,
                      const float* w0, const float* a_bias, float* state, float* out, int ld_out, const int* q_start,
                      const int* q_len, const int* kv_len, const int* seq_slot, int n_seqs, int H, int dk, int dv,
                      cudaStream_t s) {
  if (n_seqs <= 0) return 0;
#define B2B_DELTA(R)                                                                                                    \
  return launch_delta_r<R>(proj, ld, off_r, off_k, off_v, off_a, lora, ld_l, w0, a_bias, state, out, ld_out, q_start,   \
                           q_len, kv_len, seq_slot, n_seqs, H, dk, dv, s)
  if (dk <= 16) B2B_DELTA(2);
  if (dk <= 32) B2B_DELTA(4);
  if (dk <= 64) B2B_DELTA(8);
  if (dk <= 128) B2B_DELTA(16);
  if (dk <= 256) B2B_DELTA(32);
#undef B2B_DELTA
  return -2;
}

int launch_delta_post(const float* o, int ld_o, const float* gate, int ld_g, int off_g, const float* weight, void* out,
                      int ld_out, int T, int H, int dv, float eps, int f32, cudaStream_t s) {
  const long long warps = static_cast<long long>(T) * H;
  if (warps <= 0) return 0;
  const int blocks = static_cast<int>((warps + 3) / 4);
  if (f32)
    delta_post_kernel<float><<<blocks, 128, 0, s>>>(o, ld_o, gate, ld_g, off_g, weight, static_cast<float*>(out), ld_out,
                                                    T, H, dv, eps);
  else
    delta_post_kernel<bf16><<<blocks, 128, 0, s>>>(o, ld_o, gate, ld_g, off_g, weight, static_cast<bf16*>(out), ld_out, T,
                                                   H, dv, eps);
  return last_error();
}

}  // namespace b2b
