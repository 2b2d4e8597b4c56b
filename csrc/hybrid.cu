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

#include "launch.cuh"

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

// Programmatic dependent launch, as every kernel of the step does it: let the next kernel of the stream become resident
// now (it blocks in its own wait), then wait until everything launched before this kernel has completed and is visible.
__device__ __forceinline__ void pdl_begin() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

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
// streams[t, s, :] = scale * table[id] + pair[(prev * mul_prev + id * mul_cur) % buckets]   (row `buckets` at position 0)
// for every stream s.  The previous token of a span's first token comes from the sequence state (prev_tok[slot]).
// grid (token chunks, sequences).
template <typename WT>
__global__ void hyb_embed_kernel(const int* __restrict__ ids, const int* __restrict__ positions,
                                 const int* __restrict__ q_start, const int* __restrict__ q_len,
                                 const int* __restrict__ seq_slot, const int* __restrict__ prev_tok,
                                 const WT* __restrict__ table, const WT* __restrict__ pair, int buckets,
                                 long long mul_prev, long long mul_cur, float scale, float* __restrict__ streams,
                                 int ns, int W, int vocab, int tpb) {
  pdl_begin();
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
      float v = ldf(table, static_cast<size_t>(id) * W + c) * scale;
      if (row >= 0) v += ldf(pair, static_cast<size_t>(row) * W + c);
      for (int k = 0; k < ns; ++k) streams[(static_cast<size_t>(t) * ns + k) * W + c] = v;
    }
  }
}

// last token of every span -> sequence state (runs after the embedding of the step has read the old value)
__global__ void hyb_commit_prev_kernel(const int* __restrict__ ids, const int* __restrict__ q_start,
                                       const int* __restrict__ q_len, const int* __restrict__ seq_slot,
                                       int* __restrict__ prev_tok, int n_seqs) {
  pdl_begin();
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

template <int CW> struct ColVec { float v[CW]; };
template <int CW> __device__ __forceinline__ ColVec<CW> ld_cols(const float* p) {
  ColVec<CW> r;
  if constexpr (CW == 4) {
    const float4 f = *reinterpret_cast<const float4*>(p);
    r.v[0] = f.x; r.v[1] = f.y; r.v[2] = f.z; r.v[3] = f.w;
  } else {
#pragma unroll
    for (int e = 0; e < CW; ++e) r.v[e] = p[e];
  }
  return r;
}
template <int CW> __device__ __forceinline__ void st_cols(float* p, const ColVec<CW>& r) {
  if constexpr (CW == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
  } else {
#pragma unroll
    for (int e = 0; e < CW; ++e) p[e] = r.v[e];
  }
}
template <int CW> __device__ __forceinline__ void st_cols(bf16* p, const ColVec<CW>& r) {
  if constexpr (CW == 4) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(r.v[0], r.v[1]), hi = __floats2bfloat162_rn(r.v[2], r.v[3]);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&lo);
    u.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
  } else {
#pragma unroll
    for (int e = 0; e < CW; ++e) p[e] = __float2bfloat16_rn(r.v[e]);
  }
}

// NS > 0: number of streams known at compile time (no predicated slots); NS == 0: any ns <= NS_MAX.
// CW: columns per thread (4 = 128-bit accesses, needs W, ld_y, ld_h multiples of 4).
template <typename OT, int NS, int CW>
__device__ __forceinline__ void hc_row(float* __restrict__ streams, int t, int out_row, const float* __restrict__ y,
                                       int ld_y, const float* mix, const float* outw, float mult, const float* inw,
                                       const float* __restrict__ gamma, float eps, OT* __restrict__ h, int ld_h, int ns_rt,
                                       int W, int write_back, float* ubuf, float* red) {
  constexpr int NSA = NS > 0 ? NS : NS_MAX;
  const int ns = NS > 0 ? NS : ns_rt;
  float ssq = 0.f;
  for (int c = threadIdx.x * CW; c < W; c += blockDim.x * CW) {
    ColVec<CW> x[NSA];
#pragma unroll
    for (int k = 0; k < NSA; ++k)
      if (k < ns) x[k] = ld_cols<CW>(streams + (static_cast<size_t>(t) * ns + k) * W + c);
    if (y != nullptr) {
      const ColVec<CW> yv = ld_cols<CW>(y + static_cast<size_t>(t) * ld_y + c);
      ColVec<CW> nx[NSA];
#pragma unroll
      for (int j = 0; j < NSA; ++j) {
        if (j < ns) {
          const float oj = mult * outw[j];
#pragma unroll
          for (int e = 0; e < CW; ++e) {
            float a = 0.f;
#pragma unroll
            for (int k = 0; k < NSA; ++k)
              if (k < ns) a += mix[k * ns + j] * x[k].v[e];
            nx[j].v[e] = a + oj * yv.v[e];
          }
        }
      }
#pragma unroll
      for (int j = 0; j < NSA; ++j) {
        if (j < ns) {
          x[j] = nx[j];
          if (write_back) st_cols<CW>(streams + (static_cast<size_t>(t) * ns + j) * W + c, nx[j]);
        }
      }
    }
    if (gamma != nullptr) {
#pragma unroll
      for (int e = 0; e < CW; ++e) {
        float u = 0.f;
#pragma unroll
        for (int k = 0; k < NSA; ++k)
          if (k < ns) u += inw[k] * x[k].v[e];
        ubuf[c + e] = u;
        ssq += u * u;
      }
    }
  }
  if (gamma == nullptr) return;
  ssq = block_sum_(ssq, red);
  const float rinv = 1.f / sqrtf(ssq / static_cast<float>(W) + eps);
  for (int c = threadIdx.x * CW; c < W; c += blockDim.x * CW) {
    ColVec<CW> o;
#pragma unroll
    for (int e = 0; e < CW; ++e) o.v[e] = ubuf[c + e] * rinv * (1.f + gamma[c + e]);
    st_cols<CW>(h + static_cast<size_t>(out_row) * ld_h + c, o);
  }
}

// rows given by (sequence, token-in-span): grid (token chunks, sequences)
template <typename OT, int NS, int CW>
__global__ void __launch_bounds__(256) hc_step_kernel(float* streams, const int* __restrict__ q_start, const int* __restrict__ q_len,
                               const int* __restrict__ rows, const float* y, int ld_y, const float* __restrict__ mix_g,
                               const float* __restrict__ outw_g, float mult, const float* __restrict__ inw_g,
                               const float* gamma, float eps, OT* h, int ld_h, int ns, int W, int tpb) {
  pdl_begin();
  extern __shared__ __align__(16) float smem[];
  float* ubuf = smem;                       // [W rounded up to 4]
  float* coef = smem + ((W + 3) & ~3);      // mix [ns*ns], out [ns], in [ns]
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
    hc_row<OT, NS, CW>(streams, rows[blockIdx.x], blockIdx.x, y, ld_y, mix, outw, mult, inw, gamma, eps, h, ld_h, ns, W, 0,
                       ubuf, red);
    return;
  }
  const int s = blockIdx.y;
  const int n = q_len[s];
  const int i0 = blockIdx.x * tpb;
  if (i0 >= n) return;
  const int t0 = q_start[s];
  const int i1 = min(n, i0 + tpb);
  for (int i = i0; i < i1; ++i) {
    hc_row<OT, NS, CW>(streams, t0 + i, t0 + i, y, ld_y, mix, outw, mult, inw, gamma, eps, h, ld_h, ns, W, 1, ubuf, red);
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------------ activations
// out[t, c] = act(in[t, off + c]) for c < n   (0 = copy, 1 = tanh, 2 = squared relu,
// 3 = xIELU: z > 0: p0 z^2 + z/2, z <= 0: p1 (e^z - 1 - z) + z/2,  4 = soft cap p0 tanh(z / p0))
template <typename OT>
__global__ void act_cols_kernel(const float* __restrict__ in, int ld_in, int off, OT* __restrict__ out, int ld_out,
                                int n, int act, float p0, float p1, size_t total) {
  pdl_begin();
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / n;
    const int c = static_cast<int>(i % n);
    float v = in[t * ld_in + off + c];
    if (act == 1) v = tanhf(v);
    else if (act == 2) { v = fmaxf(v, 0.f); v = v * v; }
    else if (act == 3) v = v > 0.f ? p0 * v * v + 0.5f * v : p1 * (expm1f(v) - v) + 0.5f * v;
    else if (act == 4) v = p0 * tanhf(v / p0);
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
  pdl_begin();
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
constexpr int SIG_MMA_MIN_Q = 16; // spans from this length on run on the tensor-core variant (bf16 mode)

template <typename CT, typename OT>
__global__ void sig_attention_kernel(const float* __restrict__ q, const CT* __restrict__ k_cache,
                                     const CT* __restrict__ v_cache, const float* __restrict__ gate, int ld_gate,
                                     int gate_off, const float* __restrict__ pb, OT* __restrict__ out, int ld_out,
                                     const int* __restrict__ block_table, int max_pages, const int* __restrict__ q_start,
                                     const int* __restrict__ q_len, const int* __restrict__ kv_len, int H, int G, int D,
                                     int V, int chunk, float scale) {
  pdl_begin();
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

// ---- tensor-core variant for spans (bf16 serving mode): S = Q K^T and O = P V as m16n8k16 bf16 MMAs with fp32
// accumulators; scores, distance bias, sigmoid and masks are computed in fp32 on the accumulator fragments, P is rounded
// to bf16 only as the operand of the second product.  A block = 64 consecutive queries of one (sequence, head), a warp =
// 16 of them; key tiles are whole KV pages (64 keys) staged in shared memory; a warp skips pages outside the position
// blocks of its rows.  DT / VT: key / value width in units of 16 channels (zero-padded in shared memory).
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ void ldsm_x2_trans(unsigned& r0, unsigned& r1, const void* p) {
  const unsigned addr = static_cast<unsigned>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr));
}
// (bf16 mode only: the result is rounded to bf16, the approximate exp / division are 1e-6 relative)
__device__ __forceinline__ float fast_sigmoid(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }

template <int DT, int VT>
__global__ void __launch_bounds__(128)
    sig_attention_mma_kernel(const float* __restrict__ q, const bf16* __restrict__ k_cache,
                             const bf16* __restrict__ v_cache, const float* __restrict__ gate, int ld_gate, int gate_off,
                             const float* __restrict__ pb, bf16* __restrict__ out, int ld_out,
                             const int* __restrict__ block_table, int max_pages, const int* __restrict__ q_start,
                             const int* __restrict__ q_len, const int* __restrict__ kv_len, int H, int G, int D, int V,
                             int chunk, float scale) {
  pdl_begin();
  constexpr int DP = 16 * DT, VP = 16 * VT, KS = DP + 8, VS = VP + 8;
  __shared__ __align__(16) bf16 Ks[64 * KS];
  __shared__ __align__(16) bf16 Vs[64 * VS];
  const int s = blockIdx.z, hd = blockIdx.y, n = q_len[s];
  const int ib = blockIdx.x * 64;
  if (ib >= n) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
  const int t0 = q_start[s], pos0 = kv_len[s] - n;
  const int g = hd / (H / G);
  const int i_r0 = ib + warp * 16 + gid, i_r1 = i_r0 + 8;
  const bool ok0 = i_r0 < n, ok1 = i_r1 < n;
  const int p0 = pos0 + i_r0, p1 = pos0 + i_r1;
  const int lo0 = chunk > 0 ? (p0 / chunk) * chunk : 0, lo1 = chunk > 0 ? (p1 / chunk) * chunk : 0;
  const int pfirst = pos0 + ib, pmax = pos0 + min(n, ib + 64) - 1;
  const int lo_min = chunk > 0 ? (pfirst / chunk) * chunk : 0;
  const int wi0 = ib + warp * 16;
  const bool wact = wi0 < n;
  const int wpmin = pos0 + wi0, wpmax = pos0 + min(n - 1, wi0 + 15);
  const int wlo = chunk > 0 ? (wpmin / chunk) * chunk : 0;
  unsigned qa[DT][4];
  {
    const float* q0 = q + (static_cast<size_t>(t0 + (ok0 ? i_r0 : ib)) * H + hd) * D;
    const float* q1 = q + (static_cast<size_t>(t0 + (ok1 ? i_r1 : ib)) * H + hd) * D;
#pragma unroll
    for (int kk = 0; kk < DT; ++kk) {
      const int c0 = kk * 16 + 2 * tig, c1 = c0 + 8;
      const bool a = c0 < D, b = c1 < D;
      qa[kk][0] = (ok0 && a) ? pack_bf16x2(q0[c0] * scale, q0[c0 + 1] * scale) : 0u;
      qa[kk][1] = (ok1 && a) ? pack_bf16x2(q1[c0] * scale, q1[c0 + 1] * scale) : 0u;
      qa[kk][2] = (ok0 && b) ? pack_bf16x2(q0[c1] * scale, q0[c1 + 1] * scale) : 0u;
      qa[kk][3] = (ok1 && b) ? pack_bf16x2(q1[c1] * scale, q1[c1 + 1] * scale) : 0u;
    }
  }
  float oacc[2 * VT][4];
#pragma unroll
  for (int vt = 0; vt < 2 * VT; ++vt) oacc[vt][0] = oacc[vt][1] = oacc[vt][2] = oacc[vt][3] = 0.f;
  const float slope = exp2f(-8.f * static_cast<float>(hd + 1) / static_cast<float>(H));
  const float bias = pb[hd];
  const int* bt = block_table + static_cast<size_t>(s) * max_pages;
  for (int pg = lo_min >> 6; pg <= (pmax >> 6); ++pg) {
    const size_t page = static_cast<size_t>(bt[pg]);
    const int kb = pg * 64;
    __syncthreads();                           // every warp is done with the previous tile
    {
      const bf16* ksrc = k_cache + (page * 64 * G + g) * D;
      const bf16* vsrc = v_cache + (page * 64 * G + g) * V;
      constexpr int KC = DP / 8, VC = VP / 8;
      for (int idx = threadIdx.x; idx < 64 * KC; idx += 128) {
        const int r = idx / KC, c8 = idx % KC;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (c8 * 8 < D) v = *reinterpret_cast<const uint4*>(ksrc + static_cast<size_t>(r) * G * D + c8 * 8);
        *reinterpret_cast<uint4*>(Ks + r * KS + c8 * 8) = v;
      }
      for (int idx = threadIdx.x; idx < 64 * VC; idx += 128) {
        const int r = idx / VC, c8 = idx % VC;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (c8 * 8 < V) v = *reinterpret_cast<const uint4*>(vsrc + static_cast<size_t>(r) * G * V + c8 * 8);
        *reinterpret_cast<uint4*>(Vs + r * VS + c8 * 8) = v;
      }
    }
    __syncthreads();
    if (!wact || kb > wpmax || kb + 63 < wlo) continue;      // warp-uniform: no key of this page is visible to the warp
    float sc[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
      const bf16* krow = Ks + (nt * 8 + gid) * KS + 2 * tig;
#pragma unroll
      for (int kk = 0; kk < DT; ++kk) {
        const unsigned b0 = *reinterpret_cast<const unsigned*>(krow + kk * 16);
        const unsigned b1 = *reinterpret_cast<const unsigned*>(krow + kk * 16 + 8);
        mma_bf16_16816(sc[nt], qa[kk], b0, b1);
      }
    }
    unsigned pa[4][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int j0 = kb + nt * 8 + 2 * tig, j1 = j0 + 1;
      const float w00 = (ok0 && j0 >= lo0 && j0 <= p0) ? fast_sigmoid(sc[nt][0] - slope * static_cast<float>(p0 - j0) + bias) : 0.f;
      const float w01 = (ok0 && j1 >= lo0 && j1 <= p0) ? fast_sigmoid(sc[nt][1] - slope * static_cast<float>(p0 - j1) + bias) : 0.f;
      const float w10 = (ok1 && j0 >= lo1 && j0 <= p1) ? fast_sigmoid(sc[nt][2] - slope * static_cast<float>(p1 - j0) + bias) : 0.f;
      const float w11 = (ok1 && j1 >= lo1 && j1 <= p1) ? fast_sigmoid(sc[nt][3] - slope * static_cast<float>(p1 - j1) + bias) : 0.f;
      pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16x2(w00, w01);
      pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16x2(w10, w11);
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const bf16* vrow = Vs + (kk * 16 + (lane & 15)) * VS;
#pragma unroll
      for (int vt = 0; vt < 2 * VT; ++vt) {
        unsigned b0, b1;
        ldsm_x2_trans(b0, b1, vrow + vt * 8);
        mma_bf16_16816(oacc[vt], pa[kk], b0, b1);
      }
    }
  }
  if (!wact) return;
#pragma unroll
  for (int vt = 0; vt < 2 * VT; ++vt) {
    const int col = vt * 8 + 2 * tig;
    if (col >= V) continue;
    if (ok0) {
      const size_t t = static_cast<size_t>(t0 + i_r0);
      const float* gr = gate + t * ld_gate + gate_off + hd * V + col;
      const unsigned o = pack_bf16x2(oacc[vt][0] * fast_sigmoid(gr[0]), oacc[vt][1] * fast_sigmoid(gr[1]));
      *reinterpret_cast<unsigned*>(out + t * ld_out + hd * V + col) = o;
    }
    if (ok1) {
      const size_t t = static_cast<size_t>(t0 + i_r1);
      const float* gr = gate + t * ld_gate + gate_off + hd * V + col;
      const unsigned o = pack_bf16x2(oacc[vt][2] * fast_sigmoid(gr[0]), oacc[vt][3] * fast_sigmoid(gr[1]));
      *reinterpret_cast<unsigned*>(out + t * ld_out + hd * V + col) = o;
    }
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
constexpr int DL_COLS = 32;      // state columns per block
// Columns per thread: every decay / key / receptance value read from shared memory serves that many columns (with one
// column per thread the scan is bound by shared-memory bandwidth; with many, too few warps are left to hide the latency
// of the token-sequential chain).  Spans: 2; decode steps: 4 with 16-byte state accesses.
template <bool DEC> struct DeltaCpt { static constexpr int value = DEC ? 4 : 2; };

// R: key channels per thread, LN: lanes that share a column group (key channels padded to R * LN).
// Spans (DEC = false): the block has LN * 32 / C scan threads plus DL_STAGE_THREADS staging threads.  While the scan
// warps walk through tile i (the only token-sequential work), the staging warps fetch the projections of tile i + 1 and
// turn them into decay / removal rate / unit key in the other half of a double buffer -- the exponentials, divisions and
// global-load latency are off the critical path; one block barrier per tile.
// Decode steps (DEC = true): every span is one token; all threads stage, then scan: a stream over the states.
constexpr int DL_STAGE_THREADS = 128;

// CB: state columns per block (fewer columns = more blocks when heads x sequences alone do not fill the machine)
template <int R, int LN, bool DEC, int CB>
__global__ void __launch_bounds__(LN* CB / DeltaCpt<DEC>::value + (DEC ? 0 : DL_STAGE_THREADS))
    delta_scan_kernel(const float* __restrict__ proj, int ld, int off_r, int off_k, int off_v, int off_a,
                      const float* __restrict__ lora, int ld_l, const float* __restrict__ w0,
                      const float* __restrict__ a_bias, float* __restrict__ state, float* __restrict__ out, int ld_out,
                      const int* __restrict__ q_start, const int* __restrict__ q_len, const int* __restrict__ kv_len,
                      const int* __restrict__ seq_slot, int H, int dk, int dv) {
  pdl_begin();
  constexpr int C = DeltaCpt<DEC>::value;
  constexpr int NSCAN = LN * CB / C;               // scan threads
  constexpr int NSTW = DEC ? NSCAN / 32 : DL_STAGE_THREADS / 32;   // staging warps
  constexpr int DKP = R * LN;
  constexpr int EPL = (DKP + 31) / 32;             // key channels per lane while staging
  constexpr int TPW = DEC ? 1 : (DKP <= 128 ? 2 : 1);   // tokens per staging warp and tile
  constexpr int TT = NSTW * TPW;                   // tokens per tile
  constexpr int NBUF = DEC ? 1 : 2;
  __shared__ __align__(16) float rs[NBUF * TT * DKP];
  __shared__ __align__(16) float ks[NBUF * TT * DKP];
  __shared__ __align__(16) float ws[NBUF * TT * DKP];
  __shared__ __align__(16) float aus[NBUF * TT * DKP];
  __shared__ __align__(16) float us[NBUF * TT * DKP];
  __shared__ __align__(16) float vs[NBUF * TT * CB];
  const int s = blockIdx.z, hd = blockIdx.y;
  const int n = q_len[s];
  if (n <= 0) return;                               // (block-uniform)
  const int t0 = q_start[s];
  const int pos0 = kv_len[s] - n;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool scanner = DEC || tid < NSCAN;
  const bool stager = DEC || tid >= NSCAN;
  const int sw = DEC ? warp : warp - NSCAN / 32;    // staging warp index
  const int cgp = (tid % NSCAN) / LN, l = tid % LN;
  const int c0 = blockIdx.x * CB + cgp * C;    // first of this thread's C columns
  const bool vec = C == 4 && (dv % 4 == 0) && (c0 + C <= dv);        // 16-byte state accesses
  float* S_g = state + (static_cast<size_t>(seq_slot[s]) * H + hd) * static_cast<size_t>(dk) * dv;
  // key channel owned by (lane l, register m): groups of 4 channels are dealt round-robin to the LN lanes, so the lanes of
  // a column group read consecutive 16-byte words of shared memory (no bank conflicts)
  auto chan = [&](int m) { return R >= 4 ? ((m >> 2) * LN + l) * 4 + (m & 3) : l + LN * m; };
  float S[C][R];
  if (scanner) {
#pragma unroll
    for (int m = 0; m < R; ++m) {
      const int i = chan(m);
      const bool ld_ok = pos0 > 0 && i < dk;
      if (vec) {
        float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (ld_ok) v4 = *reinterpret_cast<const float4*>(S_g + static_cast<size_t>(i) * dv + c0);
        const float v[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int c = 0; c < C; ++c) S[c][m] = v[c & 3];
      } else {
#pragma unroll
        for (int c = 0; c < C; ++c) S[c][m] = (ld_ok && c0 + c < dv) ? S_g[static_cast<size_t>(i) * dv + c0 + c] : 0.f;
      }
    }
  }
  const float decay_c = 0.60653065971263342f;      // e^(-1/2)
  float w0r[EPL], abr[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    const int i = lane + 32 * e;
    w0r[e] = (stager && i < dk) ? w0[hd * dk + i] : 0.f;
    abr[e] = (stager && i < dk) ? a_bias[hd * dk + i] : 0.f;
  }
  float pr[TPW][EPL], pk[TPW][EPL], pl[TPW][EPL], pa[TPW][EPL], pv[TPW];
  const int vc = blockIdx.x * CB + lane;
  auto load_tile = [&](int tb) {                   // staging warps: raw projections of TPW tokens -> registers
#pragma unroll
    for (int tw = 0; tw < TPW; ++tw) {
      const int tt = sw * TPW + tw;
      const bool tok = tb + tt < n;
      const size_t t = static_cast<size_t>(t0 + tb + (tok ? tt : 0));
      const float* prow = proj + t * ld + hd * dk;
      const float* lrow = lora + t * ld_l + hd * dk;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const int i = lane + 32 * e;
        const bool ok = tok && i < dk;
        pr[tw][e] = ok ? prow[off_r + i] : 0.f;
        pk[tw][e] = ok ? prow[off_k + i] : 0.f;
        pl[tw][e] = ok ? lrow[i] : 0.f;
        pa[tw][e] = ok ? prow[off_a + i] : 0.f;
      }
      pv[tw] = (tok && lane < CB && vc < dv) ? proj[t * ld + off_v + hd * dv + vc] : 0.f;
    }
  };
  auto stage_tile = [&](int buf) {                 // ... -> decay, removal * unit key, unit key in shared memory
#pragma unroll
    for (int tw = 0; tw < TPW; ++tw) {
      const int tt = buf * TT + sw * TPW + tw;
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) ss += pk[tw][e] * pk[tw][e];
      ss = warp_sum_(ss);
      const float rinv = 1.f / sqrtf(ss + 1e-6f);
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const int i = lane + 32 * e;
        if (i < DKP) {
          const bool ok = i < dk;
          const float uv = pk[tw][e] * rinv;
          rs[tt * DKP + i] = pr[tw][e];
          ks[tt * DKP + i] = pk[tw][e];
          ws[tt * DKP + i] = ok ? expf(-decay_c * sigmoidf_(pl[tw][e] + w0r[e])) : 0.f;
          aus[tt * DKP + i] = ok ? sigmoidf_(pa[tw][e] + abr[e]) * uv : 0.f;
          us[tt * DKP + i] = uv;
        }
      }
      if (lane < CB) vs[tt * CB + lane] = pv[tw];
    }
  };
  auto scan_tile = [&](int buf, int tb, int nt) {
    // only u^T S sits on the token-to-token critical path; the partial outputs of the whole tile are reduced over the
    // lanes afterwards (independent shuffle trees)
    float po[TT][C];
#pragma unroll
    for (int tl = 0; tl < TT; ++tl) {
      if (tl >= nt) break;
      const int tt = buf * TT + tl;
      float vj[C], part[C], o[C];
#pragma unroll
      for (int c = 0; c < C; ++c) {
        vj[c] = vs[tt * CB + cgp * C + c];
        part[c] = 0.f;
        o[c] = 0.f;
      }
      if constexpr (R >= 4) {
        const int o4 = tt * (DKP / 4) + l;
#pragma unroll
        for (int m4 = 0; m4 < R / 4; ++m4) {
          const float4 u4 = reinterpret_cast<const float4*>(us)[o4 + m4 * LN];
#pragma unroll
          for (int c = 0; c < C; ++c)
            part[c] += (u4.x * S[c][4 * m4] + u4.y * S[c][4 * m4 + 1]) + (u4.z * S[c][4 * m4 + 2] + u4.w * S[c][4 * m4 + 3]);
        }
#pragma unroll
        for (int sh = 1; sh < LN; sh *= 2)
#pragma unroll
          for (int c = 0; c < C; ++c) part[c] += __shfl_xor_sync(0xffffffffu, part[c], sh);
#pragma unroll
        for (int m4 = 0; m4 < R / 4; ++m4) {
          const float4 w4 = reinterpret_cast<const float4*>(ws)[o4 + m4 * LN];
          const float4 a4 = reinterpret_cast<const float4*>(aus)[o4 + m4 * LN];
          const float4 k4 = reinterpret_cast<const float4*>(ks)[o4 + m4 * LN];
          const float4 r4 = reinterpret_cast<const float4*>(rs)[o4 + m4 * LN];
#pragma unroll
          for (int c = 0; c < C; ++c) {
            S[c][4 * m4] = w4.x * S[c][4 * m4] - a4.x * part[c] + k4.x * vj[c];
            S[c][4 * m4 + 1] = w4.y * S[c][4 * m4 + 1] - a4.y * part[c] + k4.y * vj[c];
            S[c][4 * m4 + 2] = w4.z * S[c][4 * m4 + 2] - a4.z * part[c] + k4.z * vj[c];
            S[c][4 * m4 + 3] = w4.w * S[c][4 * m4 + 3] - a4.w * part[c] + k4.w * vj[c];
            o[c] += (S[c][4 * m4] * r4.x + S[c][4 * m4 + 1] * r4.y) + (S[c][4 * m4 + 2] * r4.z + S[c][4 * m4 + 3] * r4.w);
          }
        }
      } else {
#pragma unroll
        for (int m = 0; m < R; ++m) {
          const float uv = us[tt * DKP + l + LN * m];
#pragma unroll
          for (int c = 0; c < C; ++c) part[c] += uv * S[c][m];
        }
#pragma unroll
        for (int sh = 1; sh < LN; sh *= 2)
#pragma unroll
          for (int c = 0; c < C; ++c) part[c] += __shfl_xor_sync(0xffffffffu, part[c], sh);
#pragma unroll
        for (int m = 0; m < R; ++m) {
          const int o1 = tt * DKP + l + LN * m;
          const float wv = ws[o1], av = aus[o1], kv = ks[o1], rv = rs[o1];
#pragma unroll
          for (int c = 0; c < C; ++c) {
            S[c][m] = wv * S[c][m] - av * part[c] + kv * vj[c];
            o[c] += S[c][m] * rv;
          }
        }
      }
#pragma unroll
      for (int c = 0; c < C; ++c) po[tl][c] = o[c];
    }
#pragma unroll
    for (int tl = 0; tl < TT; ++tl) {
      if (tl >= nt) break;
#pragma unroll
      for (int sh = 1; sh < LN; sh *= 2)
#pragma unroll
        for (int c = 0; c < C; ++c) po[tl][c] += __shfl_xor_sync(0xffffffffu, po[tl][c], sh);
      if (l == 0) {
        float* orow = out + static_cast<size_t>(t0 + tb + tl) * ld_out + hd * dv + c0;
#pragma unroll
        for (int c = 0; c < C; ++c)
          if (c0 + c < dv) orow[c] = po[tl][c];
      }
    }
  };
  if constexpr (DEC) {
    load_tile(0);
    stage_tile(0);
    __syncthreads();
    scan_tile(0, 0, min(TT, n));
  } else {
    const int ntiles = (n + TT - 1) / TT;
    if (stager) {
      load_tile(0);
      stage_tile(0);
    }
    __syncthreads();
    for (int it = 0; it < ntiles; ++it) {
      const int tb = it * TT;
      if (scanner) {
        scan_tile(it & 1, tb, min(TT, n - tb));
      } else if (it + 1 < ntiles) {
        load_tile(tb + TT);
        stage_tile((it + 1) & 1);
      }
      __syncthreads();               // tile it + 1 is staged, tile it is consumed (every thread runs ntiles rounds)
    }
  }
  if (scanner) {
#pragma unroll
    for (int m = 0; m < R; ++m) {
      const int i = chan(m);
      if (i >= dk) continue;
      if (vec) {
        *reinterpret_cast<float4*>(S_g + static_cast<size_t>(i) * dv + c0) =
            make_float4(S[0][m], S[1 % C][m], S[2 % C][m], S[3 % C][m]);
      } else {
#pragma unroll
        for (int c = 0; c < C; ++c)
          if (c0 + c < dv) S_g[static_cast<size_t>(i) * dv + c0 + c] = S[c][m];
      }
    }
  }
}

// o [T, H*dv] fp32 -> per head: o / sqrt(mean(o^2) + eps) * weight * sigmoid(gate)   -> AT.  One warp per (token, head).
template <typename OT>
__global__ void delta_post_kernel(const float* __restrict__ o, int ld_o, const float* __restrict__ gate, int ld_g,
                                  int off_g, const float* __restrict__ weight, OT* __restrict__ out, int ld_out, int T,
                                  int H, int dv, float eps) {
  pdl_begin();
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
                     long long mul_cur, float scale, float* streams, int ns, int W, int vocab, int n_seqs, int max_q,
                     int f32, cudaStream_t s) {
  if (n_seqs <= 0 || max_q <= 0) return 0;
  const int tpb = 4;
  dim3 grid((max_q + tpb - 1) / tpb, n_seqs);
  if (f32)
    launch_kernel(hyb_embed_kernel<float>, dim3(grid), dim3(256), 0, s, 1u, ids, positions, q_start, q_len, seq_slot, prev_tok,
                                                 static_cast<const float*>(table), static_cast<const float*>(pair),
                                                 buckets, mul_prev, mul_cur, scale, streams, ns, W, vocab, tpb);
  else
    launch_kernel(hyb_embed_kernel<bf16>, dim3(grid), dim3(256), 0, s, 1u, ids, positions, q_start, q_len, seq_slot, prev_tok,
                                                static_cast<const bf16*>(table), static_cast<const bf16*>(pair), buckets,
                                                mul_prev, mul_cur, scale, streams, ns, W, vocab, tpb);
  return last_error();
}

int launch_hyb_commit_prev(const int* ids, const int* q_start, const int* q_len, const int* seq_slot, int* prev_tok,
                           int n_seqs, cudaStream_t s) {
  if (n_seqs <= 0) return 0;
  launch_kernel(hyb_commit_prev_kernel, dim3((n_seqs + 127) / 128), dim3(128), 0, s, 1u, ids, q_start, q_len, seq_slot, prev_tok, n_seqs);
  return last_error();
}

template <typename OT, int NS, int CW>
static void hc_launch(dim3 grid, size_t smem, cudaStream_t s, float* streams, const int* q_start, const int* q_len,
                      const int* rows, const float* y, int ld_y, const float* mix, const float* outw, float mult,
                      const float* inw, const float* gamma, float eps, void* h, int ld_h, int ns, int W, int tpb) {
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(hc_step_kernel<OT, NS, CW>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  launch_kernel(hc_step_kernel<OT, NS, CW>, dim3(grid), dim3(256), smem, s, 1u, streams, q_start, q_len, rows, y, ld_y, mix, outw, mult, inw, gamma,
                                                     eps, static_cast<OT*>(h), ld_h, ns, W, tpb);
}

template <typename OT, int CW>
static void hc_dispatch(int ns, dim3 grid, size_t smem, cudaStream_t s, float* streams, const int* q_start,
                        const int* q_len, const int* rows, const float* y, int ld_y, const float* mix, const float* outw,
                        float mult, const float* inw, const float* gamma, float eps, void* h, int ld_h, int W, int tpb) {
#define B2B_HC(N)                                                                                                       \
  case N:                                                                                                               \
    hc_launch<OT, N, CW>(grid, smem, s, streams, q_start, q_len, rows, y, ld_y, mix, outw, mult, inw, gamma, eps, h,    \
                         ld_h, ns, W, tpb);                                                                             \
    break;
  switch (ns) {
    B2B_HC(1) B2B_HC(2) B2B_HC(3) B2B_HC(4) B2B_HC(5) B2B_HC(6) B2B_HC(8)
    default:
      hc_launch<OT, 0, CW>(grid, smem, s, streams, q_start, q_len, rows, y, ld_y, mix, outw, mult, inw, gamma, eps, h,
                           ld_h, ns, W, tpb);
  }
#undef B2B_HC
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
  const size_t smem = (static_cast<size_t>((W + 3) & ~3) + ns * ns + 2 * ns) * sizeof(float);
  const bool vec = W % 4 == 0 && (y == nullptr || ld_y % 4 == 0) && (h == nullptr || ld_h % 4 == 0);
  if (f32) {
    if (vec) hc_dispatch<float, 4>(ns, grid, smem, s, streams, q_start, q_len, rows, y, ld_y, mix, outw, mult, inw, gamma, eps, h, ld_h, W, tpb);
    else hc_dispatch<float, 1>(ns, grid, smem, s, streams, q_start, q_len, rows, y, ld_y, mix, outw, mult, inw, gamma, eps, h, ld_h, W, tpb);
  } else {
    if (vec) hc_dispatch<bf16, 4>(ns, grid, smem, s, streams, q_start, q_len, rows, y, ld_y, mix, outw, mult, inw, gamma, eps, h, ld_h, W, tpb);
    else hc_dispatch<bf16, 1>(ns, grid, smem, s, streams, q_start, q_len, rows, y, ld_y, mix, outw, mult, inw, gamma, eps, h, ld_h, W, tpb);
  }
  return last_error();
}

int launch_act_cols(const float* in, int ld_in, int off, void* out, int ld_out, int n, int act, float p0, float p1, int T,
                    int f32, cudaStream_t s) {
  const size_t total = static_cast<size_t>(T) * n;
  if (total == 0) return 0;
  const int blocks = static_cast<int>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
  if (f32) launch_kernel(act_cols_kernel<float>, dim3(blocks), dim3(256), 0, s, 1u, in, ld_in, off, static_cast<float*>(out), ld_out, n, act, p0, p1, total);
  else launch_kernel(act_cols_kernel<bf16>, dim3(blocks), dim3(256), 0, s, 1u, in, ld_in, off, static_cast<bf16*>(out), ld_out, n, act, p0, p1, total);
  return last_error();
}

int launch_attn_prep(const float* proj, int ld, const float* qn, const float* kn, const int* slots, float* q_out,
                     void* k_cache, void* v_cache, int T, int H, int G, int D, int V, float eps, int f32,
                     cudaStream_t s) {
  const long long warps = static_cast<long long>(T) * (H + 2 * G);
  if (warps <= 0) return 0;
  const int blocks = static_cast<int>((warps + 3) / 4);
  if (f32)
    launch_kernel(attn_prep_kernel<float>, dim3(blocks), dim3(128), 0, s, 1u, proj, ld, qn, kn, slots, q_out, static_cast<float*>(k_cache),
                                                   static_cast<float*>(v_cache), T, H, G, D, V, eps);
  else
    launch_kernel(attn_prep_kernel<bf16>, dim3(blocks), dim3(128), 0, s, 1u, proj, ld, qn, kn, slots, q_out, static_cast<bf16*>(k_cache),
                                                  static_cast<bf16*>(v_cache), T, H, G, D, V, eps);
  return last_error();
}

int launch_sig_attention(const float* q, const void* k_cache, const void* v_cache, const float* gate, int ld_gate,
                         int gate_off, const float* pb, void* out, int ld_out, const int* block_table, int max_pages,
                         const int* q_start, const int* q_len, const int* kv_len, int n_seqs, int max_q, int H, int G,
                         int D, int V, int chunk, float scale, int f32, cudaStream_t s) {
  if (n_seqs <= 0 || max_q <= 0) return 0;
  if (V > 32 * ATT_VR || G <= 0 || H % G != 0) return -2;
  if (!f32 && max_q >= SIG_MMA_MIN_Q && D % 8 == 0 && V % 8 == 0 && D <= 128 && V <= 128 && ld_out % 2 == 0) {
    dim3 mgrid((max_q + 63) / 64, H, n_seqs);
    const int dt = D <= 32 ? 2 : (D <= 64 ? 4 : 8), vt = V <= 32 ? 2 : (V <= 64 ? 4 : 8);
#define B2B_SIGMMA(A, B)                                                                                                \
  if (dt == A && vt == B)                                                                                               \
    launch_kernel(sig_attention_mma_kernel<A, B>, dim3(mgrid), dim3(128), 0, s, 1u,                                                                \
        q, static_cast<const bf16*>(k_cache), static_cast<const bf16*>(v_cache), gate, ld_gate, gate_off, pb,           \
        static_cast<bf16*>(out), ld_out, block_table, max_pages, q_start, q_len, kv_len, H, G, D, V, chunk, scale);
    B2B_SIGMMA(2, 2) B2B_SIGMMA(2, 4) B2B_SIGMMA(2, 8) B2B_SIGMMA(4, 2) B2B_SIGMMA(4, 4) B2B_SIGMMA(4, 8)
    B2B_SIGMMA(8, 2) B2B_SIGMMA(8, 4) B2B_SIGMMA(8, 8)
#undef B2B_SIGMMA
    return last_error();
  }
  dim3 grid((max_q + ATT_WARPS - 1) / ATT_WARPS, H, n_seqs);
  const size_t smem = static_cast<size_t>(ATT_WARPS) * D * sizeof(float);
  if (f32)
    launch_kernel(sig_attention_kernel<float, float>, dim3(grid), dim3(32 * ATT_WARPS), smem, s, 1u, 
        q, static_cast<const float*>(k_cache), static_cast<const float*>(v_cache), gate, ld_gate, gate_off, pb,
        static_cast<float*>(out), ld_out, block_table, max_pages, q_start, q_len, kv_len, H, G, D, V, chunk, scale);
  else
    launch_kernel(sig_attention_kernel<bf16, bf16>, dim3(grid), dim3(32 * ATT_WARPS), smem, s, 1u, 
        q, static_cast<const bf16*>(k_cache), static_cast<const bf16*>(v_cache), gate, ld_gate, gate_off, pb,
        static_cast<bf16*>(out), ld_out, block_table, max_pages, q_start, q_len, kv_len, H, G, D, V, chunk, scale);
  return last_error();
}

template <int R, int LN, bool DEC, int CB>
static int launch_delta_cb(const float* proj, int ld, int off_r, int off_k, int off_v, int off_a, const float* lora,
                           int ld_l, const float* w0, const float* a_bias, float* state, float* out, int ld_out,
                           const int* q_start, const int* q_len, const int* kv_len, const int* seq_slot, int n_seqs, int H,
                           int dk, int dv, cudaStream_t s) {
  dim3 grid((dv + CB - 1) / CB, H, n_seqs);
  launch_kernel(delta_scan_kernel<R, LN, DEC, CB>, dim3(grid),
                dim3(LN * CB / DeltaCpt<DEC>::value + (DEC ? 0 : DL_STAGE_THREADS)), 0, s, 1u, proj, ld, off_r, off_k, off_v,
                off_a, lora, ld_l, w0, a_bias, state, out, ld_out, q_start, q_len, kv_len, seq_slot, H, dk, dv);
  return last_error();
}

template <int R, int LN, bool DEC>
static int launch_delta_r(const float* proj, int ld, int off_r, int off_k, int off_v, int off_a, const float* lora,
                          int ld_l, const float* w0, const float* a_bias, float* state, float* out, int ld_out,
                          const int* q_start, const int* q_len, const int* kv_len, const int* seq_slot, int n_seqs, int H,
                          int dk, int dv, cudaStream_t s) {
#define B2B_CB(CB)                                                                                                      \
  return launch_delta_cb<R, LN, DEC, CB>(proj, ld, off_r, off_k, off_v, off_a, lora, ld_l, w0, a_bias, state, out,      \
                                         ld_out, q_start, q_len, kv_len, seq_slot, n_seqs, H, dk, dv, s)
  if constexpr (!DEC) {
    // the scan of a span is sequential in its tokens: its only parallelism is heads x sequences x column blocks, so
    // narrow the column blocks until about one block per SM exists
    const long long heads = static_cast<long long>(H) * n_seqs;
    if (heads * ((dv + 31) / 32) < 120 && dv > 8) {
      if (heads * ((dv + 15) / 16) >= 120 || dv <= 16) B2B_CB(16);
      B2B_CB(8);
    }
  }
  B2B_CB(32);
#undef B2B_CB
}

int launch_delta_scan(const float* proj, int ld, int off_r, int off_k, int off_v, int off_a, const float* lora, int ld_l,
                      const float* w0, const float* a_bias, float* state, float* out, int ld_out, const int* q_start,
                      const int* q_len, const int* kv_len, const int* seq_slot, int n_seqs, int max_q, int H, int dk, int dv,
                      cudaStream_t s) {
  if (n_seqs <= 0) return 0;
  // (key channels per thread, lanes per column group); a block = 32 columns x LN / 4 threads
#define B2B_DELTA(R, LN, DEC)                                                                                           \
  return launch_delta_r<R, LN, DEC>(proj, ld, off_r, off_k, off_v, off_a, lora, ld_l, w0, a_bias, state, out, ld_out,   \
                                    q_start, q_len, kv_len, seq_slot, n_seqs, H, dk, dv, s)
  if (max_q <= 1) {
    if (dk <= 16) B2B_DELTA(2, 8, true);
    if (dk <= 32) B2B_DELTA(4, 8, true);
    if (dk <= 64) B2B_DELTA(4, 16, true);
    if (dk <= 128) B2B_DELTA(8, 16, true);
    if (dk <= 256) B2B_DELTA(16, 16, true);
  } else {
    if (dk <= 16) B2B_DELTA(2, 8, false);
    if (dk <= 32) B2B_DELTA(4, 8, false);
    if (dk <= 64) B2B_DELTA(4, 16, false);
    if (dk <= 128) B2B_DELTA(8, 16, false);
    if (dk <= 256) B2B_DELTA(16, 16, false);
  }
#undef B2B_DELTA
  return -2;
}

int launch_delta_post(const float* o, int ld_o, const float* gate, int ld_g, int off_g, const float* weight, void* out,
                      int ld_out, int T, int H, int dv, float eps, int f32, cudaStream_t s) {
  const long long warps = static_cast<long long>(T) * H;
  if (warps <= 0) return 0;
  const int blocks = static_cast<int>((warps + 3) / 4);
  if (f32)
    launch_kernel(delta_post_kernel<float>, dim3(blocks), dim3(128), 0, s, 1u, o, ld_o, gate, ld_g, off_g, weight, static_cast<float*>(out), ld_out,
                                                    T, H, dv, eps);
  else
    launch_kernel(delta_post_kernel<bf16>, dim3(blocks), dim3(128), 0, s, 1u, o, ld_o, gate, ld_g, off_g, weight, static_cast<bf16*>(out), ld_out, T,
                                                   H, dv, eps);
  return last_error();
}

}  // namespace b2b
