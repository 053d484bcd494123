// Latent attention: every token caches ONE row shared by all heads, a normed latent c [rank] and a rotated key
// part kr [rot], in pages of two planes ([page_size, rank] then [page_size, rot] per page). With the per-head key
// up-projection folded into the query (qa_h = W_uk,h^T q_h, made by a batched product before this kernel) a head's
// score against key j is (qa_h . c_j + qr_h . kr_j) * scale, and its output is W_uv,h (sum_j p_j c_j): the kernel
// only ever reads the cached rows, each once for all the heads of a group.
//
//   latent_prepare    per token: rotates the rot part of every query head in place and, for a layer that owns its
//                     cache, norms the latent (x / rms * weight) and rotates the shared key part into the pages.
//                     Angles are position * inv_freq[i], made in double so that they are exact to float32; pair i is
//                     the entries (i, i + dims/2) or, with `neighbours`, (2i, 2i + 1); cosines and sines are
//                     multiplied by `magnitude` (1 unless the frequencies were rescaled for longer contexts).
//   latent_attention  one block per (token, group of heads): causal, optionally the last `window` keys only,
//                     softmax in float32 kept online per warp and merged through shared memory; the result is the
//                     attention-weighted latent times sigmoid(gate) of the head (the gate is a scalar per head, so it
//                     commutes with the value up-projection that follows).
//   steps of few tokens  (decoding) cut every token's keys into runs that separate blocks take and a merge kernel
//                     joins: in bfloat16 on the tensor cores, a block per token with all its heads (up to 32) as the
//                     rows of the products (`latent_decode_mma_kernel`), else on CUDA cores with a lane per key.
#include "common.cuh"
#include "mma_util.cuh"

// Cache of one layer: page p holds plane 0 at p * page_elems, plane 1 at p * page_elems + page_size * rank.
template <typename TA>
__global__ void latent_prepare_kernel(TA* __restrict__ q, long long q_stride, const TA* __restrict__ dkv,
                                      long long dkv_stride, const float* __restrict__ latent_norm_w,
                                      const double* __restrict__ inv_freq, const int* __restrict__ positions,
                                      const int* __restrict__ token_req, const int* __restrict__ table,
                                      int table_width, TA* __restrict__ cache, int page_size, int n_heads, int dn,
                                      int dr, int rot_dims, int rank, float eps, int neighbours, float magnitude) {
  extern __shared__ float sm[];
  float* cs = sm;                       // [rot_dims / 2] cosines, then as many sines
  float* sn = sm + rot_dims / 2;
  __shared__ float red[33];
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = rot_dims / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double s, c;
    sincos((double)pos * inv_freq[i], &s, &c);
    cs[i] = (float)c * magnitude;
    sn[i] = (float)s * magnitude;
  }
  __syncthreads();
  // Pair i is the entries (i, i + half), or with `neighbours` the entries (2i, 2i + 1).
  const int first = neighbours ? 2 : 1, apart = neighbours ? 1 : half;
  TA* qt = q + (size_t)t * q_stride;
  for (int e = threadIdx.x; e < n_heads * half; e += blockDim.x) {
    const int h = e / half, i = e % half;
    TA* p = qt + (size_t)h * (dn + dr) + dn + first * i;
    const float u = to_float(p[0]), v = to_float(p[apart]);
    p[0] = from_float<TA>(u * cs[i] - v * sn[i]);
    p[apart] = from_float<TA>(v * cs[i] + u * sn[i]);
  }
  if (dkv == nullptr) return;
  const TA* row = dkv + (size_t)t * dkv_stride;
  float ss = 0.f;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    const float x = to_float(row[c]);
    ss += x * x;
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)rank + eps);
  int page = table[(size_t)token_req[t] * table_width + pos / page_size];
  page = LLMRS_CHECKED_PAGE(page, 2, t);
  const int slot = pos % page_size;
  TA* pc = cache + (size_t)page * page_size * (rank + dr);
  TA* c_out = pc + (size_t)slot * rank;
  TA* r_out = pc + (size_t)page_size * rank + (size_t)slot * dr;
  for (int c = threadIdx.x; c < rank; c += blockDim.x)
    c_out[c] = from_float<TA>(to_float(row[c]) * inv * latent_norm_w[c]);
  const TA* kr = row + rank;
  for (int i = threadIdx.x; i < dr; i += blockDim.x) {
    float x;
    if (i >= rot_dims) x = to_float(kr[i]);
    else if (neighbours) {
      const int j = i >> 1;
      x = (i & 1) ? to_float(kr[i]) * cs[j] + to_float(kr[i - 1]) * sn[j]
                  : to_float(kr[i]) * cs[j] - to_float(kr[i + 1]) * sn[j];
    } else if (i < half) x = to_float(kr[i]) * cs[i] - to_float(kr[i + half]) * sn[i];
    else x = to_float(kr[i]) * cs[i - half] + to_float(kr[i - half]) * sn[i - half];
    r_out[i] = from_float<TA>(x);
  }
}

LLMRS_API int llmrs_latent_prepare(void* q, long long q_stride, const void* dkv, long long dkv_stride, int dtype,
                                   const float* latent_norm_w, const double* inv_freq, const int* positions,
                                   const int* token_req, const int* table, int table_width, void* cache,
                                   int page_size, int n_tokens, int n_heads, int dn, int dr, int rot_dims, int rank,
                                   float eps, int neighbours, float magnitude, cudaStream_t stream) {
  LLMRS_REQUIRE(n_tokens >= 0 && n_heads > 0 && dn >= 0 && dr > 0 && rank > 0, "latent_prepare: bad sizes");
  LLMRS_REQUIRE(rot_dims % 2 == 0 && rot_dims >= 0 && rot_dims <= dr, "latent_prepare: %d rotated dimensions of %d",
                rot_dims, dr);
  LLMRS_REQUIRE(dkv == nullptr || (cache && table && latent_norm_w), "latent_prepare: a cache write needs its pages");
  if (n_tokens == 0) return 0;
  const size_t smem = (size_t)rot_dims * sizeof(float);
  if (dtype == LLMRS_F32)
    latent_prepare_kernel<float><<<n_tokens, 128, smem, stream>>>(
        (float*)q, q_stride, (const float*)dkv, dkv_stride, latent_norm_w, inv_freq, positions, token_req, table,
        table_width, (float*)cache, page_size, n_heads, dn, dr, rot_dims, rank, eps, neighbours, magnitude);
  else if (dtype == LLMRS_BF16)
    latent_prepare_kernel<__nv_bfloat16><<<n_tokens, 128, smem, stream>>>(
        (__nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)dkv, dkv_stride, latent_norm_w, inv_freq, positions,
        token_req, table, table_width, (__nv_bfloat16*)cache, page_size, n_heads, dn, dr, rot_dims, rank, eps,
        neighbours, magnitude);
  else
    return llmrs_fail("latent_prepare: unknown dtype %d", dtype);
  return llmrs_launch_status("latent_prepare");
}

// ---------------------------------------------------------------------------------
// The attention itself. HG heads per block share every cached row; a lane holds elements lane, lane + 32, ... of a row
// (MAXC of them for the latent). Four warps take the keys in turn.
// ---------------------------------------------------------------------------------
constexpr int LA_WARPS = 4;

template <typename TA, int HG, int MAXC>
__global__ void __launch_bounds__(LA_WARPS * 32)
latent_attention_kernel(const TA* __restrict__ qa, long long qa_token, long long qa_head,
                        const TA* __restrict__ q, long long q_stride, int q_rot_at, int q_head_width,
                        const TA* __restrict__ gate, long long gate_stride, const TA* __restrict__ cache,
                        const int* __restrict__ table, int table_width, const int* __restrict__ positions,
                        const int* __restrict__ token_req, TA* __restrict__ out, long long out_token,
                        long long out_head, int n_heads, int rank, int dr, int page_size, int window, float scale,
                        int split_keys, float* __restrict__ partial) {
  extern __shared__ float sm[];
  float* s_qr = sm;                                        // [HG][dr]
  float* s_m = s_qr + HG * dr;                             // [warps][HG]
  float* s_l = s_m + LA_WARPS * HG;                        // [warps][HG]
  float* s_acc = s_l + LA_WARPS * HG;                      // [warps][HG][rank]
  const int t = blockIdx.x, h0 = blockIdx.y * HG;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pos = positions[t];
  const int* tab = table + (size_t)token_req[t] * table_width;
  int lo = window > 0 ? max(0, pos - window + 1) : 0;
  int hi = pos;
  if (partial != nullptr) {       // this block's share of the keys; it may be empty
    lo += blockIdx.z * split_keys;
    hi = min(pos, lo + split_keys - 1);
  }

  float qv[HG][MAXC], acc[HG][MAXC], m[HG], l[HG];
#pragma unroll
  for (int g = 0; g < HG; ++g) {
    const int h = min(h0 + g, n_heads - 1);
    const TA* qrow = qa + (size_t)t * qa_token + (size_t)h * qa_head;
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      const int c = lane + 32 * i;
      qv[g][i] = c < rank ? to_float(qrow[c]) : 0.f;
      acc[g][i] = 0.f;
    }
    m[g] = -INFINITY, l[g] = 0.f;
    const TA* qr = q + (size_t)t * q_stride + (size_t)h * q_head_width + q_rot_at;
    for (int i = threadIdx.x; i < dr; i += blockDim.x) s_qr[g * dr + i] = to_float(qr[i]);
  }
  __syncthreads();
  const size_t page_elems = (size_t)page_size * (rank + dr);
  for (int j = lo + warp; j <= hi; j += LA_WARPS) {
    int page = tab[j / page_size];
    page = LLMRS_CHECKED_PAGE(page, 3, j);
    const int slot = j % page_size;
    const TA* crow = cache + (size_t)page * page_elems + (size_t)slot * rank;
    const TA* rrow = cache + (size_t)page * page_elems + (size_t)page_size * rank + (size_t)slot * dr;
    float cv[MAXC];
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      const int c = lane + 32 * i;
      cv[i] = c < rank ? to_float(crow[c]) : 0.f;
    }
    float part[HG];
#pragma unroll
    for (int g = 0; g < HG; ++g) {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < MAXC; ++i) s = fmaf(qv[g][i], cv[i], s);
      part[g] = s;
    }
    for (int i = lane; i < dr; i += 32) {
      const float kv = to_float(rrow[i]);
#pragma unroll
      for (int g = 0; g < HG; ++g) part[g] = fmaf(s_qr[g * dr + i], kv, part[g]);
    }
#pragma unroll
    for (int g = 0; g < HG; ++g) {
      const float s = warp_sum(part[g]) * scale;
      const float m_new = fmaxf(m[g], s);
      const float corr = expf(m[g] - m_new);       // exp(-inf) = 0 at the first key
      const float p = expf(s - m_new);
      l[g] = l[g] * corr + p;
      m[g] = m_new;
#pragma unroll
      for (int i = 0; i < MAXC; ++i) acc[g][i] = fmaf(p, cv[i], acc[g][i] * corr);
    }
  }
  // Merge the warps' partial softmaxes.
#pragma unroll
  for (int g = 0; g < HG; ++g) {
    if (lane == 0) s_m[warp * HG + g] = m[g], s_l[warp * HG + g] = l[g];
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      const int c = lane + 32 * i;
      if (c < rank) s_acc[(size_t)(warp * HG + g) * rank + c] = acc[g][i];
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < HG * rank; e += blockDim.x) {
    const int g = e / rank, c = e % rank;
    if (h0 + g >= n_heads) continue;
    float mm = -INFINITY;
    for (int w = 0; w < LA_WARPS; ++w) mm = fmaxf(mm, s_m[w * HG + g]);
    float num = 0.f, den = 0.f;
    for (int w = 0; w < LA_WARPS; ++w) {
      const float mw = s_m[w * HG + g];
      if (mw == -INFINITY) continue;                // a warp that saw no key
      const float f = expf(mw - mm);
      num = fmaf(f, s_acc[(size_t)(w * HG + g) * rank + c], num);
      den = fmaf(f, s_l[w * HG + g], den);
    }
    if (partial != nullptr) {     // [token, head, split, rank + 2]: unnormalised sum, then its maximum and its weight
      float* p = partial + (((size_t)t * n_heads + h0 + g) * gridDim.z + blockIdx.z) * (rank + 2);
      p[c] = num;
      if (c == 0) p[rank] = mm, p[rank + 1] = den;
      continue;
    }
    const float gt = 1.0f / (1.0f + expf(-to_float(gate[(size_t)t * gate_stride + h0 + g])));
    out[(size_t)t * out_token + (size_t)(h0 + g) * out_head + c] = from_float<TA>(num / den * gt);
  }
}

// Merges the splits of a (token, head): out = sum_s e^(m_s - m) acc_s / sum_s e^(m_s - m) l_s, times sigmoid(gate).
template <typename TA>
__global__ void latent_combine_kernel(const float* __restrict__ partial, const TA* __restrict__ gate,
                                      long long gate_stride, TA* __restrict__ out, long long out_token,
                                      long long out_head, int n_heads, int rank, int n_splits) {
  const int t = blockIdx.x, h = blockIdx.y;
  const float* p = partial + ((size_t)t * n_heads + h) * n_splits * (rank + 2);
  float mm = -INFINITY;
  for (int s = 0; s < n_splits; ++s) mm = fmaxf(mm, p[(size_t)s * (rank + 2) + rank]);
  const float gt = 1.0f / (1.0f + expf(-to_float(gate[(size_t)t * gate_stride + h])));
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    float num = 0.f, den = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float* ps = p + (size_t)s * (rank + 2);
      if (ps[rank] == -INFINITY) continue;          // a split without keys
      const float f = expf(ps[rank] - mm);
      num = fmaf(f, ps[c], num);
      den = fmaf(f, ps[rank + 1], den);
    }
    out[(size_t)t * out_token + (size_t)h * out_head + c] = from_float<TA>(num / den * gt);
  }
}

template <typename TA, int HG>
static int launch_latent(int maxc, dim3 grid, size_t smem, cudaStream_t stream, const void* qa, long long qa_token,
                         long long qa_head, const void* q, long long q_stride, int q_rot_at, int q_head_width,
                         const void* gate, long long gate_stride, const void* cache, const int* table,
                         int table_width, const int* positions, const int* token_req, void* out, long long out_token,
                         long long out_head, int n_heads, int rank, int dr, int page_size, int window, float scale,
                         int split_keys, float* partial) {
#define LLMRS_LA(C)                                                                                                \
  latent_attention_kernel<TA, HG, C><<<grid, LA_WARPS * 32, smem, stream>>>(                                       \
      (const TA*)qa, qa_token, qa_head, (const TA*)q, q_stride, q_rot_at, q_head_width, (const TA*)gate,           \
      gate_stride, (const TA*)cache, table, table_width, positions, token_req, (TA*)out, out_token, out_head,      \
      n_heads, rank, dr, page_size, window, scale, split_keys, partial)
  if (maxc <= 2) LLMRS_LA(2);
  else if (maxc <= 4) LLMRS_LA(4);
  else if (maxc <= 8) LLMRS_LA(8);
  else LLMRS_LA(16);
#undef LLMRS_LA
  const int rc = llmrs_launch_status("latent_attention");
  if (rc != 0 || partial == nullptr) return rc;
  latent_combine_kernel<TA><<<dim3(grid.x, n_heads), 128, 0, stream>>>(partial, (const TA*)gate, gate_stride, (TA*)out,
                                                                      out_token, out_head, n_heads, rank, grid.z);
  return llmrs_launch_status("latent_attention (merge)");
}

// ---------------------------------------------------------------------------------
// Steps of few tokens (decoding): the same attention with the work laid out for latency. A warp takes 32 keys at a
// time. Scores: a lane per key walks its key's cached row in 16-byte loads against the queries of the group's heads,
// which lie in shared memory (read as broadcasts): no reduction across lanes. Values: a lane per 16-byte piece of the
// latent; the key's weight comes by shuffle, its row is read in straight 16-byte loads. The online softmax advances
// once per 32 keys. Every block leaves its partial result for the merge kernel. Needs rank and rot to be multiples of
// 16 bytes' worth of elements.
// ---------------------------------------------------------------------------------
template <typename TA> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x, v[1] = x.y, v[2] = x.z, v[3] = x.w;
  }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 x = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
      v[2 * i] = f.x, v[2 * i + 1] = f.y;
    }
  }
};

template <typename TA, int HG, int NV>      // NV: 16-byte pieces of the latent per lane (rank <= 32 * NV * Vec16::N)
__global__ void __launch_bounds__(LA_WARPS * 32)
latent_decode_kernel(const TA* __restrict__ qa, long long qa_token, long long qa_head, const TA* __restrict__ q,
                     long long q_stride, int q_rot_at, int q_head_width, const TA* __restrict__ cache,
                     const int* __restrict__ table, int table_width, const int* __restrict__ positions,
                     const int* __restrict__ token_req, int n_heads, int rank, int dr, int page_size, int window,
                     float scale, int split_keys, float* __restrict__ partial) {
  constexpr int VN = Vec16<TA>::N;
  extern __shared__ __align__(16) float sm[];
  const int KD = rank + dr;
  float* s_q = sm;                                          // [HG][KD]: folded query, then the rotated part
  float* s_m = s_q + HG * KD;                               // [warps][HG]
  float* s_l = s_m + LA_WARPS * HG;                         // [warps][HG]
  float* s_acc = s_l + LA_WARPS * HG;                       // [warps][HG][rank]
  const int t = blockIdx.x, h0 = blockIdx.y * HG;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pos = positions[t];
  const int* tab = table + (size_t)token_req[t] * table_width;
  int lo = window > 0 ? max(0, pos - window + 1) : 0;
  lo += blockIdx.z * split_keys;
  const int hi = min(pos, lo + split_keys - 1);
  for (int e = threadIdx.x; e < HG * KD; e += blockDim.x) {
    const int g = e / KD, c = e % KD, h = min(h0 + g, n_heads - 1);
    s_q[e] = c < rank ? to_float(qa[(size_t)t * qa_token + (size_t)h * qa_head + c])
                      : to_float(q[(size_t)t * q_stride + (size_t)h * q_head_width + q_rot_at + (c - rank)]);
  }
  __syncthreads();
  const size_t page_elems = (size_t)page_size * KD;
  float acc[HG][NV * VN], m[HG], l[HG];
#pragma unroll
  for (int g = 0; g < HG; ++g) {
    m[g] = -INFINITY, l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < NV * VN; ++i) acc[g][i] = 0.f;
  }
  for (int base = lo + 32 * warp; base <= hi; base += 32 * LA_WARPS) {
    const int j = base + lane;
    const bool live = j <= hi;
    const int jj = live ? j : hi;                           // idle lanes walk a real row and are masked afterwards
    int page = tab[jj / page_size];
    page = LLMRS_CHECKED_PAGE(page, 3, jj);
    const long long c_off = (long long)page * page_elems + (long long)(jj % page_size) * rank;
    const TA* crow = cache + c_off;
    const TA* rrow = cache + (size_t)page * page_elems + (size_t)page_size * rank + (size_t)(jj % page_size) * dr;
    float sc[HG];
#pragma unroll
    for (int g = 0; g < HG; ++g) sc[g] = 0.f;
    for (int c = 0; c < KD; c += VN) {
      float kv[VN];
      Vec16<TA>::load(c < rank ? crow + c : rrow + (c - rank), kv);
#pragma unroll
      for (int g = 0; g < HG; ++g) {
        const float* qg = s_q + g * KD + c;
#pragma unroll
        for (int e = 0; e < VN; e += 4) {
          const float4 q4 = *reinterpret_cast<const float4*>(qg + e);
          sc[g] = fmaf(q4.x, kv[e], fmaf(q4.y, kv[e + 1], fmaf(q4.z, kv[e + 2], fmaf(q4.w, kv[e + 3], sc[g]))));
        }
      }
    }
    float pw[HG], corr[HG];
#pragma unroll
    for (int g = 0; g < HG; ++g) {
      const float sv = live ? sc[g] * scale : -INFINITY;
      const float m_new = fmaxf(m[g], warp_max(sv));        // lane 0's key always exists: finite
      corr[g] = expf(m[g] - m_new);
      pw[g] = live ? expf(sv - m_new) : 0.f;
      l[g] = l[g] * corr[g] + warp_sum(pw[g]);
      m[g] = m_new;
#pragma unroll
      for (int i = 0; i < NV * VN; ++i) acc[g][i] *= corr[g];
    }
    const int n_live = min(32, hi - base + 1);
    for (int k = 0; k < n_live; ++k) {
      const long long off = __shfl_sync(0xffffffffu, c_off, k);
      float pk[HG];
#pragma unroll
      for (int g = 0; g < HG; ++g) pk[g] = __shfl_sync(0xffffffffu, pw[g], k);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = (i * 32 + lane) * VN;
        if (c < rank) {
          float cv[VN];
          Vec16<TA>::load(cache + off + c, cv);
#pragma unroll
          for (int g = 0; g < HG; ++g)
#pragma unroll
            for (int e = 0; e < VN; ++e) acc[g][i * VN + e] = fmaf(pk[g], cv[e], acc[g][i * VN + e]);
        }
      }
    }
  }
#pragma unroll
  for (int g = 0; g < HG; ++g) {
    if (lane == 0) s_m[warp * HG + g] = m[g], s_l[warp * HG + g] = l[g];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * 32 + lane) * VN;
      if (c < rank)
#pragma unroll
        for (int e = 0; e < VN; ++e) s_acc[(size_t)(warp * HG + g) * rank + c + e] = acc[g][i * VN + e];
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < HG * rank; e += blockDim.x) {
    const int g = e / rank, c = e % rank;
    if (h0 + g >= n_heads) continue;
    float mm = -INFINITY;
    for (int w = 0; w < LA_WARPS; ++w) mm = fmaxf(mm, s_m[w * HG + g]);
    float num = 0.f, den = 0.f;
    for (int w = 0; w < LA_WARPS; ++w) {
      const float mw = s_m[w * HG + g];
      if (mw == -INFINITY) continue;                // a warp that saw no key
      const float f = expf(mw - mm);
      num = fmaf(f, s_acc[(size_t)(w * HG + g) * rank + c], num);
      den = fmaf(f, s_l[w * HG + g], den);
    }
    float* p = partial + (((size_t)t * n_heads + h0 + g) * gridDim.z + blockIdx.z) * (rank + 2);
    p[c] = num;
    if (c == 0) p[rank] = mm, p[rank + 1] = den;
  }
}

// Launches the kernel above when the sizes allow it (returns false otherwise, having launched nothing).
template <typename TA>
static bool try_latent_decode(int* rc, dim3 grid, cudaStream_t stream, const void* qa, long long qa_token,
                              long long qa_head, const void* q, long long q_stride, int q_rot_at, int q_head_width,
                              const void* cache, const int* table, int table_width, const int* positions,
                              const int* token_req, int n_heads, int rank, int dr, int page_size, int window,
                              float scale, int split_keys, float* partial) {
  constexpr int VN = Vec16<TA>::N;
  const int hg = n_heads >= 4 ? 4 : 1;
  if (rank % VN || dr % VN || rank > 512 || ((uintptr_t)cache & 15) || (rank + dr) % 4) return false;
  const int pieces = (rank / VN + 31) / 32;                 // 16-byte pieces of the latent per lane
  if (pieces > 4 || pieces * VN * hg > 64) return false;    // at most 64 accumulators a lane
  const size_t smem = ((size_t)hg * (rank + dr) + 2 * LA_WARPS * hg + (size_t)LA_WARPS * hg * rank) * sizeof(float);
  if (smem > 48 * 1024) return false;
#define LLMRS_LD(HG_, NV_)                                                                                          \
  latent_decode_kernel<TA, HG_, NV_><<<grid, LA_WARPS * 32, smem, stream>>>(                                        \
      (const TA*)qa, qa_token, qa_head, (const TA*)q, q_stride, q_rot_at, q_head_width, (const TA*)cache, table,     \
      table_width, positions, token_req, n_heads, rank, dr, page_size, window, scale, split_keys, partial)
  if (hg == 4) {
    if (pieces == 1) LLMRS_LD(4, 1);
    else if (pieces == 2) LLMRS_LD(4, 2);
    else if (VN == 4) LLMRS_LD(4, 4);
    else return false;
  } else {
    if (pieces == 1) LLMRS_LD(1, 1);
    else if (pieces == 2) LLMRS_LD(1, 2);
    else LLMRS_LD(1, 4);
  }
#undef LLMRS_LD
  *rc = llmrs_launch_status("latent_attention (few tokens)");
  return true;
}

// ---------------------------------------------------------------------------------
// Steps of few tokens in bfloat16 on the tensor cores (mma.sync m16n8k16). A block takes ONE token and up to 16 * MT of
// its heads as the rows of the product and a run of `split_keys` keys (counted from the first visible key, rounded
// down to a multiple of 16), 16 keys at a time: a key's cached row [latent | rotated part] comes into shared memory
// once for all the heads (16-byte asynchronous copies, three buffers) and is the key operand (all rank + rot columns)
// and the value operand (the latent columns). The four warps split the k range of the score product, add their partial
// scores through shared memory, keep the same online softmax each (float32; the weights are rounded to bfloat16 as
// the value product's operand, as in the prompt kernel) and own a quarter of the latent columns each. Every block
// leaves its unnormalised sums, maximum and denominator in `partial` for the merge kernel. Needs rank % 64 == 0,
// rot % 16 == 0, pages of a multiple of 16 keys and split_keys % 16 == 0.
// ---------------------------------------------------------------------------------
constexpr int LDM_STAGES = 3;
static int g_latent_decode_mma = 1;
LLMRS_API void llmrs_latent_decode_mma(int on) { g_latent_decode_mma = on; }

template <int MT, int NTV>      // NTV: 8-column pieces of the output per warp, at most (rank / 32)
__global__ void __launch_bounds__(128)
latent_decode_mma_kernel(const __nv_bfloat16* __restrict__ qa, long long qa_token, long long qa_head,
                         const __nv_bfloat16* __restrict__ q, long long q_stride, int q_rot_at, int q_head_width,
                         const __nv_bfloat16* __restrict__ cache, const int* __restrict__ table, int table_width,
                         const int* __restrict__ positions, const int* __restrict__ token_req, int n_heads, int rank,
                         int dr, int page_size, int window, float scale, int split_keys, float* __restrict__ partial) {
  typedef __nv_bfloat16 bf16;
  constexpr int ROWS = 16 * MT;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int KD = rank + dr, LD = KD + 8;
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                          // [ROWS][LD]
  bf16* Ks = Qs + ROWS * LD;                                             // [stages][16][LD]
  float* Sp = reinterpret_cast<float*>(Ks + LDM_STAGES * 16 * LD);       // [4][ROWS][17]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int tok = blockIdx.x, h0 = blockIdx.y * ROWS, z = blockIdx.z, n_splits = gridDim.z;
  const int pos = positions[tok];
  const int* tab = table + (size_t)token_req[tok] * table_width;

  // Row r of the block is head h0 + r. Eight threads copy a row.
  for (int r = tid >> 3; r < ROWS; r += 16) {
    const int h = h0 + r;
    const bool there = h < n_heads;
    const bf16* qa_row = qa + (size_t)tok * qa_token + (size_t)(there ? h : 0) * qa_head;
    const bf16* qr_row = q + (size_t)tok * q_stride + (size_t)(there ? h : 0) * q_head_width + q_rot_at;
    bf16* dst = Qs + r * LD;
    for (int c = tid & 7; c < rank; c += 8) dst[c] = there ? qa_row[c] : __float2bfloat16_rn(0.f);
    for (int c = tid & 7; c < dr; c += 8) dst[rank + c] = there ? qr_row[c] : __float2bfloat16_rn(0.f);
  }
  bool row_there[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) row_there[mt][hf] = h0 + 16 * mt + g + 8 * hf < n_heads;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int j_first = (lo / 16) * 16 + z * split_keys;
  const int j_end = min(pos, j_first + split_keys - 1);
  const int n_tiles = j_end >= j_first ? (j_end - j_first) / 16 + 1 : 0;
  const size_t page_elems = (size_t)page_size * KD;
  const int chunks = KD / 8, c_chunks = rank / 8;
  auto load_tile = [&](int stage, int j0) {
    const int page = tab[j0 / page_size], slot0 = j0 % page_size;
    const bf16* base = cache + (size_t)(page < 0 ? 0 : page) * page_elems;
    bf16* dst = Ks + (size_t)stage * 16 * LD;
    const int key = tid >> 3;
    const bool in = page >= 0 && j0 + key <= j_end;           // later keys: zeros
    const bf16* c_src = base + (size_t)(slot0 + key) * rank;
    const bf16* r_src = base + (size_t)page_size * rank + (size_t)(slot0 + key) * dr;
    bf16* row = dst + key * LD;
    for (int ch = tid & 7; ch < c_chunks; ch += 8) cp_async_16(row + ch * 8, c_src + ch * 8, in ? 16 : 0);
    for (int ch = tid & 7; ch < chunks - c_chunks; ch += 8) cp_async_16(row + rank + ch * 8, r_src + ch * 8, in ? 16 : 0);
  };

  float acc[MT][NTV][4], m[MT][2], l[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    m[mt][0] = m[mt][1] = -INFINITY;
    l[mt][0] = l[mt][1] = 0.f;
#pragma unroll
    for (int i = 0; i < NTV; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[mt][i][e] = 0.f;
  }
  const int ntv = rank / 32, cw0 = warp * (rank / 4), k_steps = KD / 16;

  // One group of copies per tile, also where there is no tile to copy, so that the count of groups in flight is fixed.
#pragma unroll
  for (int s = 0; s < LDM_STAGES - 1; ++s) {
    if (s < n_tiles) load_tile(s, j_first + 16 * s);
    cp_async_commit();
  }
  for (int kt = 0; kt < n_tiles; ++kt) {
    const int stage = kt % LDM_STAGES, j0 = j_first + 16 * kt;
    if (kt + LDM_STAGES - 1 < n_tiles) load_tile((kt + LDM_STAGES - 1) % LDM_STAGES, j0 + 16 * (LDM_STAGES - 1));
    cp_async_commit();
    cp_async_wait<LDM_STAGES - 1>();
    __syncthreads();
    const bf16* K = Ks + (size_t)stage * 16 * LD;
    float sp[MT][2][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) sp[mt][nt][e] = 0.f;
    for (int ks = warp; ks < k_steps; ks += 4) {
      uint32_t b[2][2];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        b[nt][0] = *reinterpret_cast<const uint32_t*>(K + (nt * 8 + g) * LD + ks * 16 + 2 * t);
        b[nt][1] = *reinterpret_cast<const uint32_t*>(K + (nt * 8 + g) * LD + ks * 16 + 2 * t + 8);
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const bf16* Q = Qs + (16 * mt) * LD + ks * 16 + 2 * t;
        uint32_t a[4];
        a[0] = *reinterpret_cast<const uint32_t*>(Q + g * LD);
        a[1] = *reinterpret_cast<const uint32_t*>(Q + (g + 8) * LD);
        a[2] = *reinterpret_cast<const uint32_t*>(Q + g * LD + 8);
        a[3] = *reinterpret_cast<const uint32_t*>(Q + (g + 8) * LD + 8);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) mma_bf16_16816(sp[mt][nt], a, b[nt][0], b[nt][1]);
      }
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e)
          Sp[(warp * ROWS + 16 * mt + g + 8 * (e >> 1)) * 17 + nt * 8 + 2 * t + (e & 1)] = sp[mt][nt][e];
    __syncthreads();
    uint32_t pf[MT][4];
    float corr[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      float p[2][4];
      float row_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int hf = e >> 1, col = nt * 8 + 2 * t + (e & 1), j = j0 + col;
          float sv = 0.f;
#pragma unroll
          for (int w = 0; w < 4; ++w) sv += Sp[(w * ROWS + 16 * mt + g + 8 * hf) * 17 + col];
          const bool seen = row_there[mt][hf] && j <= j_end && j >= lo;
          sv = seen ? sv * scale : -INFINITY;
          p[nt][e] = sv;
          row_max[hf] = fmaxf(row_max[hf], sv);
        }
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        row_max[hf] = fmaxf(row_max[hf], __shfl_xor_sync(0xffffffffu, row_max[hf], 1));
        row_max[hf] = fmaxf(row_max[hf], __shfl_xor_sync(0xffffffffu, row_max[hf], 2));
        const float m_new = fmaxf(m[mt][hf], row_max[hf]);
        corr[mt][hf] = m_new == -INFINITY ? 1.f : expf(m[mt][hf] - m_new);
        float sum = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float v = m_new == -INFINITY ? 0.f : expf(p[nt][2 * hf + e] - m_new);
            p[nt][2 * hf + e] = v;
            sum += v;
          }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l[mt][hf] = l[mt][hf] * corr[mt][hf] + sum;
        m[mt][hf] = m_new;
      }
      pf[mt][0] = pack_bf16(p[0][0], p[0][1]);
      pf[mt][1] = pack_bf16(p[0][2], p[0][3]);
      pf[mt][2] = pack_bf16(p[1][0], p[1][1]);
      pf[mt][3] = pack_bf16(p[1][2], p[1][3]);
    }
    const int jm = lane >> 3;
#pragma unroll
    for (int nc = 0; nc < NTV / 2; ++nc) {
      if (2 * nc >= ntv) break;
      uint32_t b[4];
      ldmatrix_x4_trans(b, K + ((jm & 1) * 8 + (lane & 7)) * LD + cw0 + (2 * nc + (jm >> 1)) * 8);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          acc[mt][2 * nc][e] *= corr[mt][e >> 1];
          acc[mt][2 * nc + 1][e] *= corr[mt][e >> 1];
        }
        mma_bf16_16816(acc[mt][2 * nc], pf[mt], b[0], b[1]);
        mma_bf16_16816(acc[mt][2 * nc + 1], pf[mt], b[2], b[3]);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      if (!row_there[mt][hf]) continue;
      const int h = h0 + 16 * mt + g + 8 * hf;
      float* p = partial + (((size_t)tok * n_heads + h) * n_splits + z) * (rank + 2);
#pragma unroll
      for (int nt = 0; nt < NTV; ++nt) {
        if (nt >= ntv) break;
        p[cw0 + nt * 8 + 2 * t] = acc[mt][nt][2 * hf];
        p[cw0 + nt * 8 + 2 * t + 1] = acc[mt][nt][2 * hf + 1];
      }
      if (warp == 0 && t == 0) p[rank] = m[mt][hf], p[rank + 1] = l[mt][hf];
    }
}

template <int MT, int NTV>
static int launch_latent_decode_mma(dim3 grid, size_t smem, cudaStream_t stream, const void* qa, long long qa_token,
                                    long long qa_head, const void* q, long long q_stride, int q_rot_at,
                                    int q_head_width, const void* cache, const int* table, int table_width,
                                    const int* positions, const int* token_req, int n_heads, int rank, int dr,
                                    int page_size, int window, float scale, int split_keys, float* partial) {
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(latent_decode_mma_kernel<MT, NTV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return llmrs_fail("latent_attention (few tokens, tensor cores): shared memory %zu: %s", smem,
                                            cudaGetErrorString(e));
    configured = smem;
  }
  typedef __nv_bfloat16 bf16;
  latent_decode_mma_kernel<MT, NTV><<<grid, 128, smem, stream>>>(
      (const bf16*)qa, qa_token, qa_head, (const bf16*)q, q_stride, q_rot_at, q_head_width, (const bf16*)cache, table,
      table_width, positions, token_req, n_heads, rank, dr, page_size, window, scale, split_keys, partial);
  return llmrs_launch_status("latent_attention (few tokens, tensor cores)");
}

// Heads per block of the kernel above for a number of heads.
LLMRS_API int llmrs_latent_decode_mma_heads(int n_heads) { return n_heads > 16 ? 32 : 16; }

// Launches the tensor-core kernel when the sizes allow it (returns false otherwise, having launched nothing).
static bool try_latent_decode_mma(int* rc, int n_tokens, int n_splits, cudaStream_t stream, const void* qa,
                                  long long qa_token, long long qa_head, const void* q, long long q_stride,
                                  int q_rot_at, int q_head_width, const void* cache, const int* table,
                                  int table_width, const int* positions, const int* token_req, int n_heads, int rank,
                                  int dr, int page_size, int window, float scale, int split_keys, float* partial) {
  if (!g_latent_decode_mma || rank % 64 || rank > 512 || dr % 16 || page_size % 16 || split_keys % 16 ||
      ((uintptr_t)cache & 15))
    return false;
  const int rows = llmrs_latent_decode_mma_heads(n_heads), LD = rank + dr + 8;
  const size_t smem = (size_t)(rows + LDM_STAGES * 16) * LD * sizeof(__nv_bfloat16) + (size_t)4 * rows * 17 * sizeof(float);
  dim3 grid(n_tokens, (n_heads + rows - 1) / rows, n_splits);
  if (grid.y > 65535) return false;
#define LLMRS_LDM_ARGS                                                                                             \
  grid, smem, stream, qa, qa_token, qa_head, q, q_stride, q_rot_at, q_head_width, cache, table, table_width,       \
      positions, token_req, n_heads, rank, dr, page_size, window, scale, split_keys, partial
  const int ntv = rank / 32;
  if (rows == 32) {
    if (ntv <= 4) *rc = launch_latent_decode_mma<2, 4>(LLMRS_LDM_ARGS);
    else if (ntv <= 8) *rc = launch_latent_decode_mma<2, 8>(LLMRS_LDM_ARGS);
    else *rc = launch_latent_decode_mma<2, 16>(LLMRS_LDM_ARGS);
  } else {
    if (ntv <= 4) *rc = launch_latent_decode_mma<1, 4>(LLMRS_LDM_ARGS);
    else if (ntv <= 8) *rc = launch_latent_decode_mma<1, 8>(LLMRS_LDM_ARGS);
    else *rc = launch_latent_decode_mma<1, 16>(LLMRS_LDM_ARGS);
  }
#undef LLMRS_LDM_ARGS
  return true;
}

// qa: folded queries [tokens, heads, rank] with strides; q: the projected queries, head h's rotated part at
// q + t * q_stride + h * q_head_width + q_rot_at; gate: raw gate values [tokens, heads] (row stride given);
// out: [tokens, heads, rank] with strides. n_splits > 1: every (token, head group) is cut into n_splits blocks of
// split_keys keys from the first visible key on (n_splits * split_keys must cover the longest visible span), which
// leave their partial softmaxes in `partial` (float32 [tokens, heads, n_splits, rank + 2]) for a second kernel to merge.
LLMRS_API int llmrs_latent_attention(const void* qa, long long qa_token, long long qa_head, const void* q,
                                     long long q_stride, int q_rot_at, int q_head_width, const void* gate,
                                     long long gate_stride, const void* cache, int dtype, const int* table,
                                     int table_width, const int* positions, const int* token_req, void* out,
                                     long long out_token, long long out_head, int n_tokens, int n_heads, int rank,
                                     int dr, int page_size, int window, float scale, int n_splits, int split_keys,
                                     float* partial, int few_tokens, cudaStream_t stream) {
  LLMRS_REQUIRE(n_tokens >= 0 && n_heads > 0 && rank > 0 && dr > 0 && page_size > 0, "latent_attention: bad sizes");
  LLMRS_REQUIRE(rank <= 512, "latent_attention: a latent of at most 512, got %d", rank);
  LLMRS_REQUIRE(window >= 0, "latent_attention: bad window");
  if (n_tokens == 0) return 0;
  const int hg = n_heads >= 4 ? 4 : 1;
  const int maxc = (rank + 31) / 32;
  const size_t smem = ((size_t)hg * dr + 2 * LA_WARPS * hg + (size_t)LA_WARPS * hg * rank) * sizeof(float);
  LLMRS_REQUIRE(smem <= 48 * 1024, "latent_attention: sizes need %zu bytes of shared memory", smem);
  LLMRS_REQUIRE(n_splits >= 1 && n_splits <= 65535 && (n_splits == 1 || (split_keys > 0 && partial != nullptr)),
                "latent_attention: bad split");
  dim3 grid(n_tokens, (n_heads + hg - 1) / hg, n_splits);
  LLMRS_REQUIRE(grid.y <= 65535, "latent_attention: too many heads");
  if (few_tokens && partial != nullptr && split_keys > 0) {
    // The kernel laid out for latency; it always leaves partial results, which the merge kernel finishes.
    int rc = 0;
    bool done = false;
#define LLMRS_LD_ARGS                                                                                              \
  &rc, grid, stream, qa, qa_token, qa_head, q, q_stride, q_rot_at, q_head_width, cache, table, table_width,        \
      positions, token_req, n_heads, rank, dr, page_size, window, scale, split_keys, partial
    if (dtype == LLMRS_BF16)
      done = try_latent_decode_mma(&rc, n_tokens, n_splits, stream, qa, qa_token, qa_head, q, q_stride, q_rot_at,
                                   q_head_width, cache, table, table_width, positions, token_req, n_heads, rank, dr,
                                   page_size, window, scale, split_keys, partial);
    if (done) {
    } else if (dtype == LLMRS_F32) done = try_latent_decode<float>(LLMRS_LD_ARGS);
    else if (dtype == LLMRS_BF16) done = try_latent_decode<__nv_bfloat16>(LLMRS_LD_ARGS);
#undef LLMRS_LD_ARGS
    if (done) {
      if (rc != 0) return rc;
      if (dtype == LLMRS_F32)
        latent_combine_kernel<float><<<dim3(n_tokens, n_heads), 128, 0, stream>>>(
            partial, (const float*)gate, gate_stride, (float*)out, out_token, out_head, n_heads, rank, n_splits);
      else
        latent_combine_kernel<__nv_bfloat16><<<dim3(n_tokens, n_heads), 128, 0, stream>>>(
            partial, (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, out_token, out_head, n_heads, rank,
            n_splits);
      return llmrs_launch_status("latent_attention (merge)");
    }
  }
  if (n_splits == 1) partial = nullptr;
#define LLMRS_LA_ARGS                                                                                              \
  maxc, grid, smem, stream, qa, qa_token, qa_head, q, q_stride, q_rot_at, q_head_width, gate, gate_stride, cache,  \
      table, table_width, positions, token_req, out, out_token, out_head, n_heads, rank, dr, page_size, window, scale, \
      split_keys, partial
  if (dtype == LLMRS_F32) return hg == 4 ? launch_latent<float, 4>(LLMRS_LA_ARGS) : launch_latent<float, 1>(LLMRS_LA_ARGS);
  if (dtype == LLMRS_BF16)
    return hg == 4 ? launch_latent<__nv_bfloat16, 4>(LLMRS_LA_ARGS) : launch_latent<__nv_bfloat16, 1>(LLMRS_LA_ARGS);
#undef LLMRS_LA_ARGS
  return llmrs_fail("latent_attention: unknown dtype %d", dtype);
}

// ---------------------------------------------------------------------------------
// Prompt portions in bfloat16 on the tensor cores (mma.sync m16n8k16). A block takes a tile of consecutive tokens of
// one request times a group of heads as its rows, LP_MT pieces of 16 for the MMA (with two pieces: 8 tokens x 4 heads,
// or 32 tokens x 1 head) and walks the visible keys 16 at a time. A key's cached row [latent | rotated part] is copied into shared memory once
// (16-byte asynchronous copies, two buffers) and serves as the key operand (all rank + rot columns) and as the value
// operand (the latent columns). The four warps split the k range of the score product, add their partial 16 x 16
// scores through shared memory, keep the same online softmax each, and own a quarter of the latent columns of the
// output each. Needs rank % 64 == 0, rot % 16 == 0 and pages of a multiple of 16 keys.
// ---------------------------------------------------------------------------------
constexpr int LP_MT = 2;                 // 16-row pieces of a block's rows (755 us against 780 with one, rank 512, 16 heads)
constexpr int LP_ROWS = 16 * LP_MT;

template <int HG, int NTV>      // NTV: 8-column pieces of the output per warp, at most (rank / 32)
__global__ void __launch_bounds__(128)
latent_prefill_mma_kernel(const __nv_bfloat16* __restrict__ qa, long long qa_token, long long qa_head,
                          const __nv_bfloat16* __restrict__ q, long long q_stride, int q_rot_at, int q_head_width,
                          const __nv_bfloat16* __restrict__ gate, long long gate_stride,
                          const __nv_bfloat16* __restrict__ cache, const int* __restrict__ table, int table_width,
                          const int* __restrict__ positions, const int* __restrict__ token_req,
                          const int* __restrict__ tiles, __nv_bfloat16* __restrict__ out, long long out_token,
                          long long out_head, int n_heads, int rank, int dr, int page_size, int window, float scale) {
  typedef __nv_bfloat16 bf16;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int KD = rank + dr, LD = KD + 8;
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                   // [rows][LD]
  bf16* Ks = Qs + LP_ROWS * LD;                                   // [2][16][LD]
  float* Sp = reinterpret_cast<float*>(Ks + 2 * 16 * LD);         // [4][rows][17]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int t0 = tiles[2 * blockIdx.x], cnt = tiles[2 * blockIdx.x + 1], h0 = blockIdx.y * HG;
  const int p_first = positions[t0], p_last = p_first + cnt - 1;
  const int* tab = table + (size_t)token_req[t0] * table_width;

  // Row r of the block is token t0 + r / HG, head h0 + r % HG. Eight threads copy a row (no division in the loops).
  for (int r = tid >> 3; r < LP_ROWS; r += 16) {
    const int tq = r / HG, h = h0 + r % HG;
    const bool there = tq < cnt && h < n_heads;
    const bf16* qa_row = qa + (size_t)(t0 + (there ? tq : 0)) * qa_token + (size_t)(there ? h : 0) * qa_head;
    const bf16* qr_row = q + (size_t)(t0 + (there ? tq : 0)) * q_stride + (size_t)(there ? h : 0) * q_head_width + q_rot_at;
    bf16* dst = Qs + r * LD;
    for (int c = tid & 7; c < rank; c += 8) dst[c] = there ? qa_row[c] : __float2bfloat16_rn(0.f);
    for (int c = tid & 7; c < dr; c += 8) dst[rank + c] = there ? qr_row[c] : __float2bfloat16_rn(0.f);
  }
  // This lane's rows (g and g + 8 of every 16-row piece): their positions, or -1 for rows that do not exist.
  int pos_r[LP_MT][2];
#pragma unroll
  for (int mt = 0; mt < LP_MT; ++mt)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int r = 16 * mt + g + 8 * hf, tq = r / HG;
      pos_r[mt][hf] = (tq < cnt && h0 + r % HG < n_heads) ? p_first + tq : -1;
    }
  const int lo = window > 0 ? max(0, p_first - window + 1) : 0;
  const int j_begin = (lo / 16) * 16;
  const int n_tiles = (p_last - j_begin) / 16 + 1;
  const size_t page_elems = (size_t)page_size * KD;
  const int chunks = KD / 8, c_chunks = rank / 8;
  auto load_tile = [&](int stage, int j0) {
    const int page = tab[j0 / page_size], slot0 = j0 % page_size;
    const bf16* base = cache + (size_t)(page < 0 ? 0 : page) * page_elems;
    bf16* dst = Ks + (size_t)stage * 16 * LD;
    // Eight threads copy a key's row, 16 bytes at a time: first the latent, then the rotated part.
    const int key = tid >> 3;
    const bool in = page >= 0 && j0 + key <= p_last;          // later keys: zeros
    const bf16* c_src = base + (size_t)(slot0 + key) * rank;
    const bf16* r_src = base + (size_t)page_size * rank + (size_t)(slot0 + key) * dr;
    bf16* row = dst + key * LD;
    for (int ch = tid & 7; ch < c_chunks; ch += 8) cp_async_16(row + ch * 8, c_src + ch * 8, in ? 16 : 0);
    for (int ch = tid & 7; ch < chunks - c_chunks; ch += 8) cp_async_16(row + rank + ch * 8, r_src + ch * 8, in ? 16 : 0);
    cp_async_commit();
  };

  float acc[LP_MT][NTV][4], m[LP_MT][2], l[LP_MT][2];
#pragma unroll
  for (int mt = 0; mt < LP_MT; ++mt) {
    m[mt][0] = m[mt][1] = -INFINITY;
    l[mt][0] = l[mt][1] = 0.f;
#pragma unroll
    for (int i = 0; i < NTV; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[mt][i][e] = 0.f;
  }
  const int ntv = rank / 32, cw0 = warp * (rank / 4), k_steps = KD / 16;

  load_tile(0, j_begin);
  for (int kt = 0; kt < n_tiles; ++kt) {
    const int stage = kt & 1, j0 = j_begin + 16 * kt;
    if (kt + 1 < n_tiles) {
      load_tile(stage ^ 1, j0 + 16);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* K = Ks + (size_t)stage * 16 * LD;
    // Scores: this warp's share of the k range, for all rows.
    float sp[LP_MT][2][4];
#pragma unroll
    for (int mt = 0; mt < LP_MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) sp[mt][nt][e] = 0.f;
    for (int ks = warp; ks < k_steps; ks += 4) {
      uint32_t b[2][2];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        b[nt][0] = *reinterpret_cast<const uint32_t*>(K + (nt * 8 + g) * LD + ks * 16 + 2 * t);
        b[nt][1] = *reinterpret_cast<const uint32_t*>(K + (nt * 8 + g) * LD + ks * 16 + 2 * t + 8);
      }
#pragma unroll
      for (int mt = 0; mt < LP_MT; ++mt) {
        const bf16* Q = Qs + (16 * mt) * LD + ks * 16 + 2 * t;
        uint32_t a[4];
        a[0] = *reinterpret_cast<const uint32_t*>(Q + g * LD);
        a[1] = *reinterpret_cast<const uint32_t*>(Q + (g + 8) * LD);
        a[2] = *reinterpret_cast<const uint32_t*>(Q + g * LD + 8);
        a[3] = *reinterpret_cast<const uint32_t*>(Q + (g + 8) * LD + 8);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) mma_bf16_16816(sp[mt][nt], a, b[nt][0], b[nt][1]);
      }
    }
#pragma unroll
    for (int mt = 0; mt < LP_MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e)
          Sp[(warp * LP_ROWS + 16 * mt + g + 8 * (e >> 1)) * 17 + nt * 8 + 2 * t + (e & 1)] = sp[mt][nt][e];
    __syncthreads();
    // Every warp adds the four partial scores of its fragment positions and keeps the same softmax.
    uint32_t pf[LP_MT][4];
    float corr[LP_MT][2];
#pragma unroll
    for (int mt = 0; mt < LP_MT; ++mt) {
      float p[2][4];
      float row_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int hf = e >> 1, col = nt * 8 + 2 * t + (e & 1), j = j0 + col;
          float sv = 0.f;
#pragma unroll
          for (int w = 0; w < 4; ++w) sv += Sp[(w * LP_ROWS + 16 * mt + g + 8 * hf) * 17 + col];
          const int pr = pos_r[mt][hf];
          const bool seen = pr >= 0 && j <= pr && (window <= 0 || j > pr - window);
          sv = seen ? sv * scale : -INFINITY;
          p[nt][e] = sv;
          row_max[hf] = fmaxf(row_max[hf], sv);
        }
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        row_max[hf] = fmaxf(row_max[hf], __shfl_xor_sync(0xffffffffu, row_max[hf], 1));
        row_max[hf] = fmaxf(row_max[hf], __shfl_xor_sync(0xffffffffu, row_max[hf], 2));
        const float m_new = fmaxf(m[mt][hf], row_max[hf]);
        corr[mt][hf] = m_new == -INFINITY ? 1.f : expf(m[mt][hf] - m_new);
        float sum = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float v = m_new == -INFINITY ? 0.f : expf(p[nt][2 * hf + e] - m_new);
            p[nt][2 * hf + e] = v;
            sum += v;
          }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l[mt][hf] = l[mt][hf] * corr[mt][hf] + sum;
        m[mt][hf] = m_new;
      }
      pf[mt][0] = pack_bf16(p[0][0], p[0][1]);
      pf[mt][1] = pack_bf16(p[0][2], p[0][3]);
      pf[mt][2] = pack_bf16(p[1][0], p[1][1]);
      pf[mt][3] = pack_bf16(p[1][2], p[1][3]);
    }
    const int jm = lane >> 3;
#pragma unroll
    for (int nc = 0; nc < NTV / 2; ++nc) {
      if (2 * nc >= ntv) break;
      uint32_t b[4];
      ldmatrix_x4_trans(b, K + ((jm & 1) * 8 + (lane & 7)) * LD + cw0 + (2 * nc + (jm >> 1)) * 8);
#pragma unroll
      for (int mt = 0; mt < LP_MT; ++mt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          acc[mt][2 * nc][e] *= corr[mt][e >> 1];
          acc[mt][2 * nc + 1][e] *= corr[mt][e >> 1];
        }
        mma_bf16_16816(acc[mt][2 * nc], pf[mt], b[0], b[1]);
        mma_bf16_16816(acc[mt][2 * nc + 1], pf[mt], b[2], b[3]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int mt = 0; mt < LP_MT; ++mt)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      if (pos_r[mt][hf] < 0) continue;
      const int r = 16 * mt + g + 8 * hf, tok = t0 + r / HG, h = h0 + r % HG;
      const float gt = 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)tok * gate_stride + h])));
      const float f = gt / l[mt][hf];
      bf16* o = out + (size_t)tok * out_token + (size_t)h * out_head + cw0;
#pragma unroll
      for (int nt = 0; nt < NTV; ++nt) {
        if (nt >= ntv) break;
        *reinterpret_cast<__nv_bfloat162*>(o + nt * 8 + 2 * t) =
            __floats2bfloat162_rn(acc[mt][nt][2 * hf] * f, acc[mt][nt][2 * hf + 1] * f);
      }
    }
}

template <int HG, int NTV>
static int launch_latent_prefill(dim3 grid, size_t smem, cudaStream_t stream, const void* qa, long long qa_token,
                                 long long qa_head, const void* q, long long q_stride, int q_rot_at, int q_head_width,
                                 const void* gate, long long gate_stride, const void* cache, const int* table,
                                 int table_width, const int* positions, const int* token_req, const int* tiles,
                                 void* out, long long out_token, long long out_head, int n_heads, int rank, int dr,
                                 int page_size, int window, float scale) {
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(latent_prefill_mma_kernel<HG, NTV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return llmrs_fail("latent_attention_prefill: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = smem;
  }
  typedef __nv_bfloat16 bf16;
  latent_prefill_mma_kernel<HG, NTV><<<grid, 128, smem, stream>>>(
      (const bf16*)qa, qa_token, qa_head, (const bf16*)q, q_stride, q_rot_at, q_head_width, (const bf16*)gate,
      gate_stride, (const bf16*)cache, table, table_width, positions, token_req, tiles, (bf16*)out, out_token, out_head,
      n_heads, rank, dr, page_size, window, scale);
  return llmrs_launch_status("latent_attention_prefill");
}

// Tokens per tile of the prompt kernel for a number of heads (the tile list is made for it on the host).
LLMRS_API int llmrs_latent_prefill_tile_tokens(int n_heads) { return n_heads >= 4 ? LP_ROWS / 4 : LP_ROWS; }

// bfloat16 only. tiles: int32 [n_tiles][2] = first token of the step, tokens (at most the tile size, one request's,
// consecutive positions). Returns -2 (and launches nothing) when the sizes do not fit this kernel.
LLMRS_API int llmrs_latent_attention_prefill(const void* qa, long long qa_token, long long qa_head, const void* q,
                                             long long q_stride, int q_rot_at, int q_head_width, const void* gate,
                                             long long gate_stride, const void* cache, const int* table,
                                             int table_width, const int* positions, const int* token_req,
                                             const int* tiles, int n_tiles, void* out, long long out_token,
                                             long long out_head, int n_heads, int rank, int dr, int page_size,
                                             int window, float scale, cudaStream_t stream) {
  LLMRS_REQUIRE(n_tiles >= 0 && n_heads > 0, "latent_attention_prefill: bad sizes");
  if (rank % 64 || rank > 512 || dr % 16 || page_size % 16 || (out_token % 2) || (out_head % 2) ||
      ((uintptr_t)out & 3) || ((uintptr_t)cache & 15))
    return -2;
  if (n_tiles == 0) return 0;
  const int hg = n_heads >= 4 ? 4 : 1;
  const int LD = rank + dr + 8;
  const size_t smem = (size_t)(LP_ROWS + 2 * 16) * LD * sizeof(__nv_bfloat16) + (size_t)4 * LP_ROWS * 17 * sizeof(float);
  dim3 grid(n_tiles, (n_heads + hg - 1) / hg);
  LLMRS_REQUIRE(grid.y <= 65535, "latent_attention_prefill: too many heads");
#define LLMRS_LP_ARGS                                                                                               \
  grid, smem, stream, qa, qa_token, qa_head, q, q_stride, q_rot_at, q_head_width, gate, gate_stride, cache, table,  \
      table_width, positions, token_req, tiles, out, out_token, out_head, n_heads, rank, dr, page_size, window, scale
  const int ntv = rank / 32;
  if (hg == 4) {
    if (ntv <= 4) return launch_latent_prefill<4, 4>(LLMRS_LP_ARGS);
    if (ntv <= 8) return launch_latent_prefill<4, 8>(LLMRS_LP_ARGS);
    return launch_latent_prefill<4, 16>(LLMRS_LP_ARGS);
  }
  if (ntv <= 4) return launch_latent_prefill<1, 4>(LLMRS_LP_ARGS);
  if (ntv <= 8) return launch_latent_prefill<1, 8>(LLMRS_LP_ARGS);
  return launch_latent_prefill<1, 16>(LLMRS_LP_ARGS);
#undef LLMRS_LP_ARGS
}
