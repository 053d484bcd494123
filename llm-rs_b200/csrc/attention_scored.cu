// Attention over the paged cache with options on the score: a soft cap, a sink in the softmax's denominator, and a
// choice of masks; keys and values may have different widths.
//
//   score  = (q . k) * scale;  with softcap > 0: score = softcap * tanh(score / softcap)
//   mask   causal (key <= query), plus one of
//            window  key > query - size
//            chunk   floor(key / size) == floor(query / size), chunks counted from position 0 of the sequence
//   bias   with a table `bias` [bias_len, query heads] (float32): score += bias[min(query - key, bias_len - 1), head],
//          after the scale and the cap (a learned bias per distance, laid out per distance by the caller)
//   weights  exp(score - m) / (sum over visible keys + exp(sink_h - m)); the sink (one learned number per query head)
//            has no key and no value: it only takes weight away. Null: no sink.
//   output   the weighted sum of the values times `out_scale`
//
// A page holds, per key/value head, page_size rows of dk (keys) and then page_size rows of dv (values).
//
//   prepare   RMS norm over the WHOLE q row (all heads at once) and the whole k row with weights of that size
//             (null: no norm), rotation of the first rot_dims channels of every head (channel i with i + rot_dims/2,
//             angle position * inv_freq[i], made in double), q rewritten in place, k and v written into their pages;
//             with `unit_heads` every head of q and k is instead divided by its own root mean square AFTER the
//             rotation, without a weight;
//   head gate out[t, h, :] *= sigmoid(gate[t, h]), one number per token and query head;
//   prefill   16 queries of one request per block against the keys they may see, online softmax (any type);
//             bfloat16 with dk, dv multiples of 16 up to 128: 64 queries per block on the tensor cores (mma.sync);
//   decode    one query per request: the visible keys are cut into runs that separate blocks take, and a second
//             kernel merges the runs and adds the sink. Rows that can be read sixteen bytes a load: a block takes up
//             to four query heads of one key head together, a lane per key for the scores, lanes over channels for
//             the values. Any other size: a block per query head, a warp per key, lanes over channels.
// Scores, weights and sums are float32.
#include "common.cuh"
#include "mma_util.cuh"

enum { MASK_CAUSAL = 0, MASK_WINDOW = 1, MASK_CHUNK = 2 };

struct ScoreOpts {
  float scale, softcap;
  const float* sink;
  int mask, size;
  const float* bias;      // [bias_len, bias_heads] or null
  int bias_len, bias_heads;
  float out_scale;
};
// The bias of a key `dist` positions behind its query, for one query head.
__device__ __forceinline__ float dist_bias(const ScoreOpts& o, int head, int dist) {
  return o.bias[(size_t)min(max(dist, 0), o.bias_len - 1) * o.bias_heads + min(head, o.bias_heads - 1)];
}

__device__ __forceinline__ int first_visible(const ScoreOpts& o, int pos) {
  if (o.mask == MASK_WINDOW) return max(0, pos - o.size + 1);
  if (o.mask == MASK_CHUNK) return (pos / o.size) * o.size;
  return 0;
}
__device__ __forceinline__ float capped(const ScoreOpts& o, float s) {
  s *= o.scale;
  return o.softcap > 0.f ? o.softcap * tanhf(s / o.softcap) : s;
}
// For the tensor-core kernel: 2^x and 1/x by the hardware's approximations (relative errors 2^-22 and one unit in the
// last place), and the soft cap built on them, cap * tanh(s / cap) = cap - 2 cap / (2^(2 s log2(e) / cap) + 1), in the
// softmax's base-2 scale: a product, an exponential, a sum, a reciprocal and a fused multiply-add per score. The absolute
// error is that of a float32 number of the cap's size (the subtraction from cap rounds there whatever the method); all of
// it is float32 arithmetic. The kernel for any type keeps tanhf and expf.
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_fast(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
struct FastCap {
  float in, out;      // score * in -> exponent; cap * log2(e) = out
  bool on;
  __device__ __forceinline__ FastCap(const ScoreOpts& o) {
    constexpr float LOG2E = 1.4426950408889634f;
    on = o.softcap > 0.f;
    in = on ? o.scale * 2.0f * LOG2E / o.softcap : o.scale * LOG2E;
    out = o.softcap * LOG2E;
  }
  // The capped score times log2(e).
  __device__ __forceinline__ float operator()(float s) const {
    const float t = s * in;
    if (!on) return t;
    return fmaf(rcp_fast(ex2_fast(fminf(t, 80.0f)) + 1.0f), -2.0f * out, out);
  }
};
__device__ __host__ __forceinline__ size_t page_head_offset(int page, int kvh, int n_kv_heads, int page_size, int dk,
                                                            int dv) {
  return ((size_t)page * n_kv_heads + kvh) * (size_t)page_size * (dk + dv);
}

// ---------------------------------------------------------------------------------
// prepare
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void scored_prepare_kernel(T* __restrict__ q, long long q_stride, const T* __restrict__ k,
                                      long long k_stride, const T* __restrict__ v, long long v_stride,
                                      const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w,
                                      const double* __restrict__ inv_freq, const int* __restrict__ positions,
                                      const int* __restrict__ token_req, const int* __restrict__ block_table,
                                      int table_stride, T* __restrict__ cache, int n_q_heads, int n_kv_heads, int dk,
                                      int dv, int rot_dims, int page_size, float eps, int unit_heads, int unit_values,
                                      const T* __restrict__ v_first, long long v_first_stride,
                                      const float* __restrict__ v_mix) {
  extern __shared__ float sm[];
  __shared__ float red[33];
  const int t = blockIdx.x, pos = positions[t];
  const int wq = n_q_heads * dk, wk = k ? n_kv_heads * dk : 0, half = rot_dims / 2;
  float* xq = sm;              // [wq]
  float* xk = xq + wq;         // [wk]
  float* cs = xk + wk;         // [half][2]
  float sq = 0.f, sk = 0.f;
  for (int c = threadIdx.x; c < wq; c += blockDim.x) {
    const float f = to_float(q[(size_t)t * q_stride + c]);
    xq[c] = f;
    sq = fmaf(f, f, sq);
  }
  for (int c = threadIdx.x; c < wk; c += blockDim.x) {
    const float f = to_float(k[(size_t)t * k_stride + c]);
    xk[c] = f;
    sk = fmaf(f, f, sk);
  }
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double s, c;
    sincos((double)pos * inv_freq[i], &s, &c);
    cs[2 * i] = (float)c;
    cs[2 * i + 1] = (float)s;
  }
  sq = block_sum(sq, red);
  sk = block_sum(sk, red);
  const float inv_q = q_norm_w ? 1.0f / sqrtf(sq / (float)wq + eps) : 1.0f;
  const float inv_k = (k_norm_w && wk) ? 1.0f / sqrtf(sk / (float)wk + eps) : 1.0f;
  auto turned = [&](const float* x, const float* w, float inv, int head, int i) {
    const int c = head * dk + i;
    float a = x[c] * inv * (w ? w[c] : 1.0f);
    if (i < rot_dims) {
      const int j = i < half ? i : i - half;
      const int pc = head * dk + (i < half ? i + half : i - half);
      const float b = x[pc] * inv * (w ? w[pc] : 1.0f);
      a = i < half ? a * cs[2 * j] - b * cs[2 * j + 1] : a * cs[2 * j] + b * cs[2 * j + 1];
    }
    return a;
  };
  // The values as the pages keep them: with `unit_values` every head's value divided by its own root mean square (no
  // weight), then with `v_first` mixed with another layer's values of the same token, (1 - m) v + m v_first.
  auto write_values = [&](int page, int slot) {
    const float mix = v_first ? v_mix[0] : 0.f;
    auto mixed = [&](float val, int c) {
      return v_first ? (1.0f - mix) * val + mix * to_float(v_first[(size_t)t * v_first_stride + c]) : val;
    };
    auto place = [&](int head, int i) {
      return page_head_offset(page, head, n_kv_heads, page_size, dk, dv) + (size_t)page_size * dk + (size_t)slot * dv + i;
    };
    if (unit_values) {
      const int lane = threadIdx.x & 31;
      for (int head = threadIdx.x >> 5; head < n_kv_heads; head += blockDim.x >> 5) {
        const T* src = v + (size_t)t * v_stride + (size_t)head * dv;
        float ss = 0.f;
        for (int i = lane; i < dv; i += 32) {
          const float f = to_float(src[i]);
          ss = fmaf(f, f, ss);
        }
        const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps);
        for (int i = lane; i < dv; i += 32)
          cache[place(head, i)] = from_float<T>(mixed(to_float(src[i]) * inv, head * dv + i));
      }
    } else if (v_first) {
      for (int c = threadIdx.x; c < n_kv_heads * dv; c += blockDim.x)
        cache[place(c / dv, c % dv)] = from_float<T>(mixed(to_float(v[(size_t)t * v_stride + c]), c));
    } else {
      for (int c = threadIdx.x; c < n_kv_heads * dv; c += blockDim.x) cache[place(c / dv, c % dv)] = v[(size_t)t * v_stride + c];
    }
  };
  if (unit_heads) {
    // Every head of q and k, AFTER its rotation, is divided by its own root mean square (no weight): a warp per head.
    const int page = k == nullptr ? 0 :
        LLMRS_CHECKED_PAGE(block_table[(size_t)token_req[t] * table_stride + pos / page_size], 2, t);
    const int slot = pos % page_size, lane = threadIdx.x & 31;
    for (int hh = threadIdx.x >> 5; hh < n_q_heads + (k ? n_kv_heads : 0); hh += blockDim.x >> 5) {
      const bool is_q = hh < n_q_heads;
      const int head = is_q ? hh : hh - n_q_heads;
      const float* x = is_q ? xq : xk;
      float ss = 0.f;
      for (int i = lane; i < dk; i += 32) {
        const float a = turned(x, nullptr, 1.0f, head, i);
        ss = fmaf(a, a, ss);
      }
      const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)dk + eps);
      T* dst = is_q ? q + (size_t)t * q_stride + (size_t)head * dk
                    : cache + page_head_offset(page, head, n_kv_heads, page_size, dk, dv) + (size_t)slot * dk;
      for (int i = lane; i < dk; i += 32) dst[i] = from_float<T>(turned(x, nullptr, 1.0f, head, i) * inv);
    }
    if (k == nullptr) return;
    write_values(page, slot);
    return;
  }
  for (int c = threadIdx.x; c < wq; c += blockDim.x)
    q[(size_t)t * q_stride + c] = from_float<T>(turned(xq, q_norm_w, inv_q, c / dk, c % dk));
  if (k == nullptr) return;
  const int page = LLMRS_CHECKED_PAGE(block_table[(size_t)token_req[t] * table_stride + pos / page_size], 2, t);
  const int slot = pos % page_size;
  for (int c = threadIdx.x; c < wk; c += blockDim.x) {
    const int head = c / dk, i = c % dk;
    cache[page_head_offset(page, head, n_kv_heads, page_size, dk, dv) + (size_t)slot * dk + i] =
        from_float<T>(turned(xk, k_norm_w, inv_k, head, i));
  }
  write_values(page, slot);
}

// q: [tokens, n_q_heads * dk] rewritten in place; k, v: the new keys and values (null: the entry reads another
// entry's pages and writes none); cache: one entry's pages. unit_values: every head's value is divided by its root mean
// square before it is kept; v_first ([tokens, n_kv_heads * dv], rows v_first_stride apart) with v_mix (one float on the
// device): the kept value is (1 - v_mix) v + v_mix v_first.
LLMRS_API int llmrs_scored_prepare(void* q, long long q_stride, const void* k, long long k_stride, const void* v,
                                   long long v_stride, int dtype, const float* q_norm_w, const float* k_norm_w,
                                   const double* inv_freq, const int* positions, const int* token_req,
                                   const int* block_table, int table_stride, void* cache, int n_tokens, int n_q_heads,
                                   int n_kv_heads, int dk, int dv, int rot_dims, int page_size, float eps,
                                   int unit_heads, int unit_values, const void* v_first, long long v_first_stride,
                                   const float* v_mix, cudaStream_t stream) {
  LLMRS_REQUIRE(n_tokens >= 0 && n_q_heads > 0 && n_kv_heads > 0 && dk > 0 && dv > 0 && page_size > 0,
                "scored_prepare: bad sizes");
  LLMRS_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dk, "scored_prepare: rot_dims %d of %d", rot_dims, dk);
  LLMRS_REQUIRE(v_first == nullptr || v_mix != nullptr, "scored_prepare: values to mix in, but no weight");
  if (n_tokens == 0) return 0;
  const size_t smem = ((size_t)(n_q_heads + n_kv_heads) * dk + rot_dims) * sizeof(float);
  LLMRS_REQUIRE(smem <= 160 * 1024, "scored_prepare: rows of %zu bytes are too wide", smem);
  const int threads = n_q_heads * dk >= 2048 ? 512 : 256;
#define LLMRS_SP_LAUNCH(T)                                                                                          \
  do {                                                                                                              \
    static size_t configured = 48 * 1024;                                                                           \
    if (smem > configured) {                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(scored_prepare_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                           (int)smem);                                                              \
      if (e != cudaSuccess) return llmrs_fail("scored_prepare: shared memory %zu: %s", smem, cudaGetErrorString(e)); \
      configured = smem;                                                                                            \
    }                                                                                                               \
    scored_prepare_kernel<T><<<n_tokens, threads, smem, stream>>>(                                                  \
        (T*)q, q_stride, (const T*)k, k_stride, (const T*)v, v_stride, q_norm_w, k_norm_w, inv_freq, positions,     \
        token_req, block_table, table_stride, (T*)cache, n_q_heads, n_kv_heads, dk, dv, rot_dims, page_size, eps,   \
        unit_heads, unit_values, (const T*)v_first, v_first_stride, v_mix);                                         \
  } while (0)
  if (dtype == LLMRS_F32) LLMRS_SP_LAUNCH(float);
  else if (dtype == LLMRS_BF16) LLMRS_SP_LAUNCH(__nv_bfloat16);
  else return llmrs_fail("scored_prepare: unknown dtype %d", dtype);
#undef LLMRS_SP_LAUNCH
  return llmrs_launch_status("scored_prepare");
}

// ---------------------------------------------------------------------------------
// head gate: out[t, h, :] *= sigmoid(gate[t, h]) (the sigmoid in float32). One block per token.
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ out, long long out_stride, const T* __restrict__ gate,
                                 long long gate_stride, int n_heads, int dv) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < n_heads * dv; c += blockDim.x) {
    const float g = 1.0f / (1.0f + expf(-to_float(gate[(size_t)t * gate_stride + c / dv])));
    T* o = out + (size_t)t * out_stride + c;
    *o = from_float<T>(to_float(*o) * g);
  }
}

LLMRS_API int llmrs_head_gate(void* out, long long out_stride, const void* gate, long long gate_stride, int dtype,
                              int n_tokens, int n_heads, int dv, cudaStream_t stream) {
  LLMRS_REQUIRE(n_tokens >= 0 && n_heads > 0 && dv > 0, "head_gate: bad sizes");
  if (n_tokens == 0) return 0;
  const int threads = n_heads * dv >= 1024 ? 256 : 128;
  if (dtype == LLMRS_F32)
    head_gate_kernel<float><<<n_tokens, threads, 0, stream>>>((float*)out, out_stride, (const float*)gate,
                                                              gate_stride, n_heads, dv);
  else if (dtype == LLMRS_BF16)
    head_gate_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
        (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)gate, gate_stride, n_heads, dv);
  else
    return llmrs_fail("head_gate: unknown dtype %d", dtype);
  return llmrs_launch_status("head_gate");
}

// ---------------------------------------------------------------------------------
// prefill, any type
// ---------------------------------------------------------------------------------
constexpr int SP_BQ = 16, SP_TILE = 64, SP_BK = 32, SP_THREADS = 256, SP_MAX_VCH = 16;

template <typename T>
__global__ void __launch_bounds__(SP_THREADS)
scored_prefill_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long out_stride,
                      const T* __restrict__ cache, const int* __restrict__ tiles, const int* __restrict__ q_start,
                      const int* __restrict__ n_new, const int* __restrict__ cached_len,
                      const int* __restrict__ block_table, int table_stride, int n_q_heads, int n_kv_heads, int dk,
                      int dv, int page_size, ScoreOpts opt) {
  extern __shared__ float smem[];
  float* Qs = smem;                       // [SP_BQ][dk]
  float* Ks = Qs + SP_BQ * dk;            // [SP_BK][dk + 1]
  float* Vs = Ks + SP_BK * (dk + 1);      // [SP_BK][dv]
  float* Ps = Vs + SP_BK * dv;            // [SP_BQ][SP_BK]
  const int tile = blockIdx.x, head = blockIdx.y;
  const int kvh = head / (n_q_heads / n_kv_heads);
  const int req = tiles[2 * tile], q_off = tiles[2 * tile + 1] + blockIdx.z * SP_BQ;
  if (q_off >= n_new[req]) return;
  const int rows = min(SP_BQ, n_new[req] - q_off);
  const int tok0 = q_start[req] + q_off;
  const int pos0 = cached_len[req] + q_off;
  const int kv_hi = pos0 + rows;
  const int key_floor = first_visible(opt, pos0);       // the first row sees furthest back; pages below may be gone
  const int kv_lo = (key_floor / SP_BK) * SP_BK;
  const int* table = block_table + (size_t)req * table_stride;
  const int tid = threadIdx.x, r = tid >> 4, c = tid & 15;

  for (int i = tid; i < SP_BQ * dk; i += SP_THREADS) {
    const int rr = i / dk, cc = i - rr * dk;
    Qs[i] = rr < rows ? to_float(q[(size_t)(tok0 + rr) * q_stride + (size_t)head * dk + cc]) : 0.f;
  }
  float acc[SP_MAX_VCH];
#pragma unroll
  for (int j = 0; j < SP_MAX_VCH; ++j) acc[j] = 0.f;
  float m = -INFINITY, l = 0.f;
  const int my_pos = pos0 + r;
  const int my_lo = first_visible(opt, my_pos);

  for (int kb = kv_lo; kb < kv_hi; kb += SP_BK) {
    __syncthreads();
    for (int i = tid; i < SP_BK * dk; i += SP_THREADS) {
      const int kk = i / dk, cc = i - kk * dk, key = kb + kk;
      float kf = 0.f;
      if (key >= key_floor && key < kv_hi) {
        const int page = LLMRS_CHECKED_PAGE(table[key / page_size], 3, key);
        kf = to_float(cache[page_head_offset(page, kvh, n_kv_heads, page_size, dk, dv) + (size_t)(key % page_size) * dk + cc]);
      }
      Ks[kk * (dk + 1) + cc] = kf;
    }
    for (int i = tid; i < SP_BK * dv; i += SP_THREADS) {
      const int kk = i / dv, cc = i - kk * dv, key = kb + kk;
      float vf = 0.f;
      if (key >= key_floor && key < kv_hi) {
        const int page = LLMRS_CHECKED_PAGE(table[key / page_size], 3, key);
        vf = to_float(cache[page_head_offset(page, kvh, n_kv_heads, page_size, dk, dv) + (size_t)page_size * dk +
                            (size_t)(key % page_size) * dv + cc]);
      }
      Vs[kk * dv + cc] = vf;
    }
    __syncthreads();
    float s[SP_BK / 16];
#pragma unroll
    for (int jj = 0; jj < SP_BK / 16; ++jj) {
      const int kk = c + 16 * jj, key = kb + kk;
      const float* qr = Qs + r * dk;
      const float* kr = Ks + kk * (dk + 1);
      float dot = 0.f;
      for (int e = 0; e < dk; ++e) dot = fmaf(qr[e], kr[e], dot);
      const bool seen = r < rows && key <= my_pos && key >= my_lo;
      s[jj] = seen ? capped(opt, dot) + (opt.bias ? dist_bias(opt, head, my_pos - key) : 0.f) : -INFINITY;
    }
    float bm = s[0];
#pragma unroll
    for (int jj = 1; jj < SP_BK / 16; ++jj) bm = fmaxf(bm, s[jj]);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, o, 16));
    const float m_new = fmaxf(m, bm);
    float corr = 1.f, bs = 0.f;
    if (m_new > -INFINITY) {
      corr = expf(m - m_new);
#pragma unroll
      for (int jj = 0; jj < SP_BK / 16; ++jj) {
        const float p = expf(s[jj] - m_new);
        Ps[r * SP_BK + c + 16 * jj] = p;
        bs += p;
      }
    } else {
#pragma unroll
      for (int jj = 0; jj < SP_BK / 16; ++jj) Ps[r * SP_BK + c + 16 * jj] = 0.f;
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) bs += __shfl_xor_sync(0xffffffffu, bs, o, 16);
    l = l * corr + bs;
    m = m_new;
    __syncwarp();
    const float* pr = Ps + r * SP_BK;
#pragma unroll
    for (int j = 0; j < SP_MAX_VCH; ++j) {
      const int col = c + 16 * j;
      if (col < dv) {
        float a = acc[j] * corr;
        for (int kk = 0; kk < SP_BK; ++kk) a = fmaf(pr[kk], Vs[kk * dv + col], a);
        acc[j] = a;
      }
    }
  }
  if (r < rows) {
    float w = 1.0f;
    if (opt.sink) {
      const float sk = opt.sink[head], mf = fmaxf(m, sk);
      w = expf(m - mf);
      l = l * w + expf(sk - mf);
    }
    const float inv = l > 0.f ? w / l * opt.out_scale : 0.f;
    T* o = out + (size_t)(tok0 + r) * out_stride + (size_t)head * dv;
#pragma unroll
    for (int j = 0; j < SP_MAX_VCH; ++j)
      if (c + 16 * j < dv) o[c + 16 * j] = from_float<T>(acc[j] * inv);
  }
}

// ---------------------------------------------------------------------------------
// prefill on the tensor cores: bfloat16, 64 queries per block (16 per warp), 64 keys per tile, two stages.
// ---------------------------------------------------------------------------------
using bf16 = __nv_bfloat16;
constexpr int SM_BQ = 64, SM_BK = 64, SM_WARPS = 4, SM_THREADS = SM_WARPS * 32;

template <int KCH, int VCH>
__global__ void __launch_bounds__(SM_THREADS, (KCH <= 8 && VCH <= 8) ? 3 : 1)
scored_prefill_mma_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out, long long out_stride,
                          const bf16* __restrict__ cache, const int* __restrict__ tiles,
                          const int* __restrict__ q_start, const int* __restrict__ n_new,
                          const int* __restrict__ cached_len, const int* __restrict__ block_table, int table_stride,
                          int n_q_heads, int n_kv_heads, int page_size, ScoreOpts opt) {
  constexpr int DK = 16 * KCH, DV = 16 * VCH, KROW = DK + 8, VROW = DV + 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* KV = reinterpret_cast<bf16*>(smem_raw);     // 2 stages x (K [64][KROW], V [64][VROW])
  constexpr int STAGE = SM_BK * (KROW + VROW);
  // The last tiles of a prompt see the most keys: they start first.
  const int head = blockIdx.x % n_q_heads;
  const int tile = (int)(gridDim.x / n_q_heads) - 1 - (int)(blockIdx.x / n_q_heads);
  const int kvh = head / (n_q_heads / n_kv_heads);
  const int req = tiles[2 * tile], q_off = tiles[2 * tile + 1];
  const int rows = min(SM_BQ, n_new[req] - q_off);
  const int tok0 = q_start[req] + q_off;
  const int pos0 = cached_len[req] + q_off;
  const int kv_hi = pos0 + rows;
  const int key_floor = first_visible(opt, pos0);        // no row reads a key below this
  const int kv_lo = (key_floor / SM_BK) * SM_BK;
  const int* table = block_table + (size_t)req * table_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gq = lane >> 2, tq = lane & 3;

  auto load_kv = [&](int kb, int stage) {
    bf16* Ks = KV + (size_t)stage * STAGE;
    bf16* Vs = Ks + SM_BK * KROW;
    for (int c = threadIdx.x; c < SM_BK * (DK / 8); c += SM_THREADS) {
      const int row = c / (DK / 8), ch = c - row * (DK / 8), key = kb + row;
      const bool valid = key >= key_floor && key < kv_hi;
      const bf16* src = cache;
      if (valid) {
        const int page = LLMRS_CHECKED_PAGE(table[key / page_size], 4, key);
        src = cache + page_head_offset(page, kvh, n_kv_heads, page_size, DK, DV) + (size_t)(key % page_size) * DK + ch * 8;
      }
      cp_async_16(Ks + row * KROW + ch * 8, src, valid ? 16 : 0);
    }
    for (int c = threadIdx.x; c < SM_BK * (DV / 8); c += SM_THREADS) {
      const int row = c / (DV / 8), ch = c - row * (DV / 8), key = kb + row;
      const bool valid = key >= key_floor && key < kv_hi;
      const bf16* src = cache;
      if (valid) {
        const int page = LLMRS_CHECKED_PAGE(table[key / page_size], 4, key);
        src = cache + page_head_offset(page, kvh, n_kv_heads, page_size, DK, DV) + (size_t)page_size * DK +
              (size_t)(key % page_size) * DV + ch * 8;
      }
      cp_async_16(Vs + row * VROW + ch * 8, src, valid ? 16 : 0);
    }
  };
  load_kv(kv_lo, 0);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  uint32_t qf[KCH][4];
  {
    const int r0 = warp * 16 + gq, r1 = r0 + 8;
    const bf16* q0 = q + (size_t)(tok0 + r0) * q_stride + (size_t)head * DK;
    const bf16* q1 = q + (size_t)(tok0 + r1) * q_stride + (size_t)head * DK;
#pragma unroll
    for (int kc = 0; kc < KCH; ++kc) {
      const int col = kc * 16 + tq * 2;
      qf[kc][0] = r0 < rows ? *reinterpret_cast<const uint32_t*>(q0 + col) : 0u;
      qf[kc][1] = r1 < rows ? *reinterpret_cast<const uint32_t*>(q1 + col) : 0u;
      qf[kc][2] = r0 < rows ? *reinterpret_cast<const uint32_t*>(q0 + col + 8) : 0u;
      qf[kc][3] = r1 < rows ? *reinterpret_cast<const uint32_t*>(q1 + col + 8) : 0u;
    }
  }
  float o[2 * VCH][4];
#pragma unroll
  for (int n = 0; n < 2 * VCH; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.f, 0.f};
  const int pos_r[2] = {pos0 + warp * 16 + gq, pos0 + warp * 16 + gq + 8};
  const int lo_r[2] = {first_visible(opt, pos_r[0]), first_visible(opt, pos_r[1])};
  const int warp_lo = first_visible(opt, pos0 + warp * 16);      // first_visible never falls as the position grows
  const int last_lo = first_visible(opt, pos0 + warp * 16 + 15);
  const FastCap cap(opt);
  constexpr float LOG2E = 1.4426950408889634f;

  int stage = 0;
  for (int kb = kv_lo; kb < kv_hi; kb += SM_BK, stage ^= 1) {
    if (kb + SM_BK < kv_hi) load_kv(kb + SM_BK, stage ^ 1);
    cp_async_commit();
    const bf16* Ks = KV + (size_t)stage * STAGE;
    const bf16* Vs = Ks + SM_BK * KROW;
    // A warp whose rows all lie before this tile, or whose rows all start after it, has nothing to add.
    const bool active = kb <= pos0 + warp * 16 + 15 && kb + SM_BK > warp_lo;
    if (active) {
      float s[SM_BK / 8][4];
#pragma unroll
      for (int n = 0; n < SM_BK / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
      for (int kc = 0; kc < KCH; ++kc) {
        const int j = lane >> 3;
#pragma unroll
        for (int np = 0; np < SM_BK / 16; ++np) {
          uint32_t b[4];
          ldmatrix_x4(b, Ks + (np * 16 + (j >> 1) * 8 + (lane & 7)) * KROW + kc * 16 + (j & 1) * 8);
          mma_bf16_16816(s[2 * np], qf[kc], b[0], b[1]);
          mma_bf16_16816(s[2 * np + 1], qf[kc], b[2], b[3]);
        }
      }
      float mx[2] = {-INFINITY, -INFINITY};
      // Only a tile that touches the diagonal, or in which some row's first visible key lies, has scores to hide.
      const int pw = pos0 + warp * 16;
      const bool need_mask = kb + SM_BK - 1 > pw || kb < last_lo;
      if (opt.bias) {
#pragma unroll
        for (int n = 0; n < SM_BK / 8; ++n)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = kb + n * 8 + tq * 2 + (e & 1);
            const bool seen = key <= pos_r[e >> 1] && key >= lo_r[e >> 1];
            s[n][e] = seen ? fmaf(dist_bias(opt, head, pos_r[e >> 1] - key), LOG2E, cap(s[n][e])) : -INFINITY;
            mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
          }
      } else if (need_mask) {
#pragma unroll
        for (int n = 0; n < SM_BK / 8; ++n)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = kb + n * 8 + tq * 2 + (e & 1);
            const bool seen = key <= pos_r[e >> 1] && key >= lo_r[e >> 1];
            s[n][e] = seen ? cap(s[n][e]) : -INFINITY;
            mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
          }
      } else {
#pragma unroll
        for (int n = 0; n < SM_BK / 8; ++n)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            s[n][e] = cap(s[n][e]);
            mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
          }
      }
      float corr[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_row[r], mx[r]);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        corr[r] = ex2_fast(m_row[r] - m_use);
        m_row[r] = m_new;
        float sum = 0.f;
#pragma unroll
        for (int n = 0; n < SM_BK / 8; ++n)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float p = ex2_fast(s[n][r * 2 + e] - m_use);
            s[n][r * 2 + e] = p;
            sum += p;
          }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l_row[r] = l_row[r] * corr[r] + sum;
      }
#pragma unroll
      for (int n = 0; n < 2 * VCH; ++n) {
        o[n][0] *= corr[0]; o[n][1] *= corr[0]; o[n][2] *= corr[1]; o[n][3] *= corr[1];
      }
#pragma unroll
      for (int kc = 0; kc < SM_BK / 16; ++kc) {
        uint32_t pf[4];
        pf[0] = pack_bf16(s[2 * kc][0], s[2 * kc][1]);
        pf[1] = pack_bf16(s[2 * kc][2], s[2 * kc][3]);
        pf[2] = pack_bf16(s[2 * kc + 1][0], s[2 * kc + 1][1]);
        pf[3] = pack_bf16(s[2 * kc + 1][2], s[2 * kc + 1][3]);
        const int j = lane >> 3;
#pragma unroll
        for (int nc = 0; nc < VCH; ++nc) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, Vs + (kc * 16 + (j & 1) * 8 + (lane & 7)) * VROW + (2 * nc + (j >> 1)) * 8);
          mma_bf16_16816(o[2 * nc], pf, b[0], b[1]);
          mma_bf16_16816(o[2 * nc + 1], pf, b[2], b[3]);
        }
      }
    }
    cp_async_wait<0>();
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + gq + r * 8;
    if (row < rows) {
      float w = 1.0f, l = l_row[r];
      if (opt.sink) {
        const float sk = opt.sink[head] * LOG2E, mf = fmaxf(m_row[r], sk);
        w = ex2_fast(m_row[r] - mf);
        l = l * w + ex2_fast(sk - mf);
      }
      const float inv = l > 0.f ? w / l * opt.out_scale : 0.f;
      bf16* orow = out + (size_t)(tok0 + row) * out_stride + (size_t)head * DV;
#pragma unroll
      for (int n = 0; n < 2 * VCH; ++n)
        *reinterpret_cast<__nv_bfloat162*>(orow + n * 8 + tq * 2) =
            __floats2bfloat162_rn(o[n][r * 2] * inv, o[n][r * 2 + 1] * inv);
    }
  }
}

template <int KCH, int VCH>
static int launch_scored_mma(const void* q, long long q_stride, void* out, long long out_stride, const void* cache,
                             const int* tiles, int n_tiles, const int* q_start, const int* n_new,
                             const int* cached_len, const int* block_table, int table_stride, int n_q_heads,
                             int n_kv_heads, int page_size, const ScoreOpts& opt, cudaStream_t stream) {
  const size_t smem = (size_t)2 * SM_BK * (16 * KCH + 8 + 16 * VCH + 8) * sizeof(bf16);
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(scored_prefill_mma_kernel<KCH, VCH>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return llmrs_fail("scored_prefill_mma: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = smem;
  }
  dim3 grid((unsigned)n_tiles * (unsigned)n_q_heads);
  scored_prefill_mma_kernel<KCH, VCH><<<grid, SM_THREADS, smem, stream>>>(
      (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)cache, tiles, q_start, n_new, cached_len,
      block_table, table_stride, n_q_heads, n_kv_heads, page_size, opt);
  return llmrs_launch_status("scored_prefill_mma");
}

// The tcgen05 kernel of attention_tc.cu (keys and values of 128 channels, long portions).
bool llmrs_attn_prefill_tc_supported(const void* q, long long q_stride, const void* cache, int d, int page_size,
                                     float scale);
int llmrs_attn_prefill_tc_scored(const void* q, long long q_stride, int n_tokens, void* out, long long out_stride,
                                 const void* cache, long long cache_rows, const int* tiles, int n_tiles,
                                 const int* q_start, const int* n_new, const int* cached_len, const int* block_table,
                                 int table_stride, int n_q_heads, int n_kv_heads, int page_size, int window, float scale,
                                 float softcap, const float* sink, int chunk, float out_scale, int* error_flag,
                                 cudaStream_t stream);

static int g_scored_generic_only = 0;
// 1: bfloat16 also takes the kernel for any type (tests compare the two).
LLMRS_API void llmrs_scored_generic_only(int on) { g_scored_generic_only = on; }

// Head sizes the tensor-core kernel is built for (keys, values), in units of 16.
#define LLMRS_SCORED_MMA_SIZES(X)                                                                              \
  X(1, 1) X(2, 2) X(3, 3) X(4, 4) X(5, 5) X(6, 6) X(7, 7) X(8, 8) X(1, 2) X(2, 1) X(2, 3) X(3, 2) X(2, 4) X(4, 2) \
  X(3, 4) X(4, 3) X(4, 6) X(6, 4) X(4, 8) X(8, 4) X(6, 8) X(8, 6) X(12, 8) X(6, 2) X(8, 2)

LLMRS_API int llmrs_scored_prefill(const void* q, long long q_stride, void* out, long long out_stride,
                                   const void* cache, const int* tiles, int n_tiles, const int* q_start,
                                   const int* n_new, const int* cached_len, const int* block_table, int table_stride,
                                   int n_q_heads, int n_kv_heads, int dk, int dv, int page_size, float scale,
                                   float softcap, const float* sink, int mask, int mask_size, const float* bias,
                                   int bias_len, float out_scale, int dtype, int n_tokens, int n_pages, int prefer_tc,
                                   cudaStream_t stream) {
  LLMRS_REQUIRE(n_tiles >= 0 && n_q_heads > 0 && n_kv_heads > 0 && page_size > 0, "scored_prefill: bad sizes");
  LLMRS_REQUIRE(n_q_heads % n_kv_heads == 0, "scored_prefill: %d query heads are no multiple of %d key heads",
                n_q_heads, n_kv_heads);
  LLMRS_REQUIRE(dk >= 1 && dk <= 256 && dv >= 1 && dv <= 16 * SP_MAX_VCH, "scored_prefill: head sizes %d / %d (1..256)",
                dk, dv);
  LLMRS_REQUIRE(mask == MASK_CAUSAL || ((mask == MASK_WINDOW || mask == MASK_CHUNK) && mask_size > 0),
                "scored_prefill: mask %d with size %d", mask, mask_size);
  LLMRS_REQUIRE(bias == nullptr || bias_len > 0, "scored_prefill: a bias table of %d rows", bias_len);
  if (n_tiles == 0) return 0;
  ScoreOpts opt{scale, softcap, sink, mask, mask_size, bias, bias_len, n_q_heads, out_scale};
  if ((long long)n_tiles * n_q_heads > 2147483647LL) return llmrs_fail("scored_prefill: %d tiles are too many", n_tiles);
  // Long portions of heads of 128 channels: the tcgen05 kernel (128-query blocks, K and V by TMA, scores in tensor
  // memory), with the cap, the sink and the mask in its softmax threads. Its waits are bounded; a block that gives
  // up leaves a code that llmrs_attention_tc_error reads.
  if (dtype == LLMRS_BF16 && prefer_tc && !g_scored_generic_only && dk == 128 && dv == 128 && n_tiles <= 8192 &&
      bias == nullptr &&
      out_stride % 8 == 0 && ((uintptr_t)out & 15) == 0 &&
      llmrs_attn_prefill_tc_supported(q, q_stride, cache, dk, page_size, scale))
    return llmrs_attn_prefill_tc_scored(q, q_stride, n_tokens, out, out_stride, cache,
                                        (long long)n_pages * n_kv_heads * 2 * page_size, tiles, n_tiles, q_start, n_new,
                                        cached_len, block_table, table_stride, n_q_heads, n_kv_heads, page_size,
                                        mask == MASK_WINDOW ? mask_size : 0, scale, softcap, sink,
                                        mask == MASK_CHUNK ? mask_size : 0, out_scale, nullptr, stream);
  if (dtype == LLMRS_BF16 && !g_scored_generic_only && q_stride % 2 == 0 && out_stride % 2 == 0) {
#define LLMRS_SM_CASE(K, V)                                                                                     \
  if (dk == 16 * K && dv == 16 * V)                                                                              \
    return launch_scored_mma<K, V>(q, q_stride, out, out_stride, cache, tiles, n_tiles, q_start, n_new,         \
                                   cached_len, block_table, table_stride, n_q_heads, n_kv_heads, page_size, opt, \
                                   stream);
    LLMRS_SCORED_MMA_SIZES(LLMRS_SM_CASE)
#undef LLMRS_SM_CASE
  }
  const size_t smem = (size_t)(SP_BQ * dk + SP_BK * (dk + 1) + SP_BK * dv + SP_BQ * SP_BK) * sizeof(float);
  dim3 grid(n_tiles, n_q_heads, SP_TILE / SP_BQ);
#define LLMRS_SPF_LAUNCH(T)                                                                                          \
  do {                                                                                                               \
    static size_t configured = 48 * 1024;                                                                            \
    if (smem > configured) {                                                                                         \
      cudaError_t e = cudaFuncSetAttribute(scored_prefill_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                           (int)smem);                                                               \
      if (e != cudaSuccess) return llmrs_fail("scored_prefill: shared memory %zu: %s", smem, cudaGetErrorString(e)); \
      configured = smem;                                                                                             \
    }                                                                                                                \
    scored_prefill_kernel<T><<<grid, SP_THREADS, smem, stream>>>(                                                    \
        (const T*)q, q_stride, (T*)out, out_stride, (const T*)cache, tiles, q_start, n_new, cached_len, block_table, \
        table_stride, n_q_heads, n_kv_heads, dk, dv, page_size, opt);                                                \
  } while (0)
  if (dtype == LLMRS_F32) LLMRS_SPF_LAUNCH(float);
  else if (dtype == LLMRS_BF16) LLMRS_SPF_LAUNCH(__nv_bfloat16);
  else return llmrs_fail("scored_prefill: unknown dtype %d", dtype);
#undef LLMRS_SPF_LAUNCH
  return llmrs_launch_status("scored_prefill");
}

// ---------------------------------------------------------------------------------
// decode
// ---------------------------------------------------------------------------------
constexpr int SD_WARPS = 4, SD_THREADS = SD_WARPS * 32, SD_MAXC = 8;      // channels per lane: head sizes up to 256
constexpr int SD_UNROLL = 4;                                               // keys a warp takes per turn

__host__ __device__ inline size_t sd_part_stride(int dv) { return (size_t)dv + 2; }

// One block per (decode request, query head, run of keys). Each warp takes four keys of every sixteen of the run: its
// lanes split the channels, the dot products are summed over the warp, the weights and the sum of values are kept online.
// Four neighbouring channels in one load (8 bytes of bfloat16, 16 of float32).
__device__ __forceinline__ void load4(const float* p, float* out) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
__device__ __forceinline__ void load4(const bf16* p, float* out) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
}

// VEC: head sizes are multiples of four and the rows aligned for it: a lane's register 4 g + e holds channel
// (lane + 32 g) * 4 + e and a row is read four channels a load. Otherwise register j holds channel lane + 32 j.
template <typename T, bool VEC>
__global__ void __launch_bounds__(SD_THREADS)
scored_decode_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ cache,
                     const int* __restrict__ dec_reqs, const int* __restrict__ q_start,
                     const int* __restrict__ cached_len, const int* __restrict__ block_table, int table_stride,
                     float* __restrict__ part, int max_splits, int split_keys, int n_q_heads, int n_kv_heads, int dk,
                     int dv, int page_size, ScoreOpts opt) {
  __shared__ float s_m[SD_WARPS], s_l[SD_WARPS];
  extern __shared__ float s_o[];      // [SD_WARPS][dv]
  const int di = blockIdx.x, head = blockIdx.y, split = blockIdx.z;
  const int kvh = head / (n_q_heads / n_kv_heads);
  const int req = dec_reqs[di];
  const int pos = cached_len[req];                  // the new token's key is in the cache already
  const int lo = first_visible(opt, pos);
  const int k_begin = lo + split * split_keys, k_end = min(k_begin + split_keys, pos + 1);
  float* pp = part + (((size_t)di * n_q_heads + head) * max_splits + split) * sd_part_stride(dv);
  if (k_begin >= k_end) {
    if (threadIdx.x == 0) { pp[0] = -INFINITY; pp[1] = 0.f; }
    return;
  }
  const int* table = block_table + (size_t)req * table_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float qr[SD_MAXC], acc[SD_MAXC];
  const T* qp = q + (size_t)q_start[req] * q_stride + (size_t)head * dk;
  auto channel = [&](int j) { return VEC ? (lane + 32 * (j >> 2)) * 4 + (j & 3) : lane + 32 * j; };
  auto load_row = [&](const T* row, int width, float* out) {
    if (VEC) {
#pragma unroll
      for (int g = 0; g < SD_MAXC / 4; ++g) {
        if ((lane + 32 * g) * 4 < width) load4(row + (lane + 32 * g) * 4, out + 4 * g);
        else out[4 * g] = out[4 * g + 1] = out[4 * g + 2] = out[4 * g + 3] = 0.f;
      }
    } else {
#pragma unroll
      for (int j = 0; j < SD_MAXC; ++j) out[j] = lane + 32 * j < width ? to_float(row[lane + 32 * j]) : 0.f;
    }
  };
  load_row(qp, dk, qr);
#pragma unroll
  for (int j = 0; j < SD_MAXC; ++j) acc[j] = 0.f;
  float m = -INFINITY, l = 0.f;
  // Four keys per turn: their rows are all asked for before the first is used, so that a warp has several loads on
  // their way (one key at a time, the kernel waited a memory round trip per key).
  for (int key0 = k_begin + warp * SD_UNROLL; key0 < k_end; key0 += SD_WARPS * SD_UNROLL) {
    float kf[SD_UNROLL][SD_MAXC], vf[SD_UNROLL][SD_MAXC];
#pragma unroll
    for (int u = 0; u < SD_UNROLL; ++u) {
      const int key = min(key0 + u, k_end - 1);
      const int page = LLMRS_CHECKED_PAGE(table[key / page_size], 3, key);
      const T* kr = cache + page_head_offset(page, kvh, n_kv_heads, page_size, dk, dv) + (size_t)(key % page_size) * dk;
      const T* vr = cache + page_head_offset(page, kvh, n_kv_heads, page_size, dk, dv) + (size_t)page_size * dk +
                    (size_t)(key % page_size) * dv;
      load_row(kr, dk, kf[u]);
      load_row(vr, dv, vf[u]);
    }
    float sc[SD_UNROLL], m_new = m;
#pragma unroll
    for (int u = 0; u < SD_UNROLL; ++u) {
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < SD_MAXC; ++j) dot = fmaf(qr[j], kf[u][j], dot);
      sc[u] = key0 + u < k_end ? capped(opt, warp_sum(dot)) + (opt.bias ? dist_bias(opt, head, pos - key0 - u) : 0.f)
                               : -INFINITY;      // the first of the four always counts
      m_new = fmaxf(m_new, sc[u]);
    }
    const float corr = expf(m - m_new);
    float p[SD_UNROLL], ps = 0.f;
#pragma unroll
    for (int u = 0; u < SD_UNROLL; ++u) {
      p[u] = expf(sc[u] - m_new);
      ps += p[u];
    }
    l = l * corr + ps;
    m = m_new;
#pragma unroll
    for (int j = 0; j < SD_MAXC; ++j) {
      float a = acc[j] * corr;
#pragma unroll
      for (int u = 0; u < SD_UNROLL; ++u) a = fmaf(p[u], vf[u][j], a);
      acc[j] = a;
    }
  }
  if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
  for (int j = 0; j < SD_MAXC; ++j)
    if (channel(j) < dv) s_o[warp * dv + channel(j)] = acc[j];
  __syncthreads();
  float mm = -INFINITY;
#pragma unroll
  for (int w = 0; w < SD_WARPS; ++w) mm = fmaxf(mm, s_m[w]);
  for (int c = threadIdx.x; c < dv; c += SD_THREADS) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < SD_WARPS; ++w) a += s_m[w] == -INFINITY ? 0.f : s_o[w * dv + c] * expf(s_m[w] - mm);
    pp[2 + c] = a;
  }
  if (threadIdx.x == 0) {
    float ll = 0.f;
#pragma unroll
    for (int w = 0; w < SD_WARPS; ++w) ll += s_m[w] == -INFINITY ? 0.f : s_l[w] * expf(s_m[w] - mm);
    pp[0] = mm;
    pp[1] = ll;
  }
}

// Sixteen bytes of a row as floats: eight bfloat16 channels or four float32 ones.
template <typename T> struct RowChunk;
template <> struct RowChunk<float> { static constexpr int N = 4; };
template <> struct RowChunk<bf16> { static constexpr int N = 8; };
__device__ __forceinline__ void load_chunk(const float* p, float* out) { load4(p, out); }
__device__ __forceinline__ void load_chunk(const bf16* p, float* out) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = __bfloat1622float2(h[i]);
    out[2 * i] = a.x;
    out[2 * i + 1] = a.y;
  }
}

// Asks for a row's 128-byte lines to be brought into the L2 (no register, no wait).
template <typename T>
__device__ __forceinline__ void prefetch_row_l2(const T* row, int width) {
  const char* p = reinterpret_cast<const char*>(row);
  const char* end = p + (size_t)width * sizeof(T);
  for (const char* line = p - ((uintptr_t)p & 127); line < end; line += 128)
    asm volatile("prefetch.global.L2 [%0];" ::"l"(line));
}

// The decode kernel for rows that can be read sixteen bytes a load: one block per (decode request, key head, up to GH
// of the query heads that share it, run of keys), so that a key and a value row are fetched once for all those heads.
// A warp takes 32 keys a turn. Scores: a LANE per key; it walks its key's row against the queries in shared memory
// (every lane reads the same query channel: a broadcast), so a score needs no sum over the warp, and the cap and the
// exponential run once per key and head, not once per lane. Values: the lanes split the channels (VG groups of 4 x 32),
// a key's weights and the place of its row come from the key's lane by shuffles.
template <typename T, int GH, int VG>
__global__ void __launch_bounds__(SD_THREADS)
scored_decode_grouped_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ cache,
                             const int* __restrict__ dec_reqs, const int* __restrict__ q_start,
                             const int* __restrict__ cached_len, const int* __restrict__ block_table,
                             int table_stride, float* __restrict__ part, int max_splits, int split_keys,
                             int n_q_heads, int n_kv_heads, int dk, int dv, int page_size, ScoreOpts opt) {
  constexpr int CW = RowChunk<T>::N;
  __shared__ float s_m[SD_WARPS][GH], s_l[SD_WARPS][GH];
  __shared__ __align__(16) float s_p[SD_WARPS][32][GH];      // a turn's weights, [key][head]
  __shared__ unsigned long long s_at[SD_WARPS][32];          // where each key's value row starts
  extern __shared__ __align__(16) float sg_smem[];      // queries [GH][dk], then the warps' sums [SD_WARPS][GH][dv]
  float* q_s = sg_smem;
  float* s_o = sg_smem + GH * dk;
  const int G = n_q_heads / n_kv_heads, hgroups = (G + GH - 1) / GH;
  const int di = blockIdx.x, kvh = blockIdx.y / hgroups, g0 = (blockIdx.y % hgroups) * GH, split = blockIdx.z;
  const int ng = min(GH, G - g0), head0 = kvh * G + g0;
  const int req = dec_reqs[di];
  const int pos = cached_len[req];                  // the new token's key is in the cache already
  const int lo = first_visible(opt, pos);
  const int k_begin = lo + split * split_keys, k_end = min(k_begin + split_keys, pos + 1);
  auto record = [&](int h) { return part + (((size_t)di * n_q_heads + head0 + h) * max_splits + split) * sd_part_stride(dv); };
  if (k_begin >= k_end) {
    if (threadIdx.x < ng) {
      float* pp = record(threadIdx.x);
      pp[0] = -INFINITY;
      pp[1] = 0.f;
    }
    return;
  }
  const int* table = block_table + (size_t)req * table_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  {
    const T* qp = q + (size_t)q_start[req] * q_stride + (size_t)head0 * dk;      // heads beyond the group: zeros
    for (int i = threadIdx.x; i < GH * dk; i += SD_THREADS) q_s[i] = i < ng * dk ? to_float(qp[i]) : 0.f;
  }
  __syncthreads();
  float acc[GH][4 * VG], m[GH], l[GH];
#pragma unroll
  for (int h = 0; h < GH; ++h) {
    m[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int j = 0; j < 4 * VG; ++j) acc[h][j] = 0.f;
  }
  const size_t head_base = (size_t)kvh * page_size * (dk + dv), page_elems = (size_t)n_kv_heads * page_size * (dk + dv);
  for (int key0 = k_begin + warp * 32; key0 < k_end; key0 += SD_WARPS * 32) {
    const bool seen = key0 + lane < k_end;
    const int key = seen ? key0 + lane : k_end - 1;
    const int page = LLMRS_CHECKED_PAGE(table[key / page_size], 3, key);
    const int row = key % page_size;
    const size_t base = (size_t)page * page_elems + head_base;
    const T* kr = cache + base + (size_t)row * dk;
    const size_t v_at = base + (size_t)page_size * dk + (size_t)row * dv;      // this lane's key's value row
    // Asked for now, the value rows of this turn and the key row of the warp's next turn are in the L2 when wanted.
    if (seen) prefetch_row_l2(cache + v_at, dv);
    if (key0 + lane + SD_WARPS * 32 < k_end) {
      const int nk = key0 + lane + SD_WARPS * 32;
      const int np = LLMRS_CHECKED_PAGE(table[nk / page_size], 3, nk);
      prefetch_row_l2(cache + (size_t)np * page_elems + head_base + (size_t)(nk % page_size) * dk, dk);
    }
    float dot[GH];
#pragma unroll
    for (int h = 0; h < GH; ++h) dot[h] = 0.f;
#pragma unroll 4
    for (int c = 0; c < dk; c += CW) {
      float kf[CW];
      load_chunk(kr + c, kf);
#pragma unroll
      for (int h = 0; h < GH; ++h) {
#pragma unroll
        for (int e = 0; e < CW; e += 4) {
          const float4 qa = *reinterpret_cast<const float4*>(q_s + h * dk + c + e);
          dot[h] = fmaf(qa.x, kf[e], dot[h]);
          dot[h] = fmaf(qa.y, kf[e + 1], dot[h]);
          dot[h] = fmaf(qa.z, kf[e + 2], dot[h]);
          dot[h] = fmaf(qa.w, kf[e + 3], dot[h]);
        }
      }
    }
    float p[GH];
#pragma unroll
    for (int h = 0; h < GH; ++h) {
      const float s = seen ? capped(opt, dot[h]) + (opt.bias ? dist_bias(opt, head0 + h, pos - key) : 0.f)
                           : -INFINITY;      // lane 0's key always counts
      const float m_new = fmaxf(m[h], warp_max(s));
      const float corr = expf(m[h] - m_new);
      p[h] = seen ? expf(s - m_new) : 0.f;
      l[h] = l[h] * corr + warp_sum(p[h]);
      m[h] = m_new;
#pragma unroll
      for (int j = 0; j < 4 * VG; ++j) acc[h][j] *= corr;
    }
    // The weights and the rows' places go through shared memory: two broadcast reads a key, where shuffles would be
    // two for the place and one per head.
    __syncwarp();
#pragma unroll
    for (int h = 0; h < GH; ++h) s_p[warp][lane][h] = p[h];
    s_at[warp][lane] = v_at;
    __syncwarp();
    const int n_here = min(32, k_end - key0);
#pragma unroll 8
    for (int u = 0; u < n_here; ++u) {
      const T* vr = cache + s_at[warp][u];
      float vf[4 * VG];
#pragma unroll
      for (int g = 0; g < VG; ++g) {
        if ((lane + 32 * g) * 4 < dv) load4(vr + (lane + 32 * g) * 4, vf + 4 * g);
        else vf[4 * g] = vf[4 * g + 1] = vf[4 * g + 2] = vf[4 * g + 3] = 0.f;
      }
#pragma unroll
      for (int h = 0; h < GH; ++h) {
        const float pu = s_p[warp][u][h];
#pragma unroll
        for (int j = 0; j < 4 * VG; ++j) acc[h][j] = fmaf(pu, vf[j], acc[h][j]);
      }
    }
  }
  // The warps' records of each head become the block's.
  if (lane == 0) {
#pragma unroll
    for (int h = 0; h < GH; ++h) { s_m[warp][h] = m[h]; s_l[warp][h] = l[h]; }
  }
#pragma unroll
  for (int h = 0; h < GH; ++h)
#pragma unroll
    for (int j = 0; j < 4 * VG; ++j) {
      const int c = (lane + 32 * (j >> 2)) * 4 + (j & 3);
      if (c < dv) s_o[((size_t)warp * GH + h) * dv + c] = acc[h][j];
    }
  __syncthreads();
  for (int i = threadIdx.x; i < ng * dv; i += SD_THREADS) {
    const int h = i / dv, c = i - h * dv;
    float mm = -INFINITY, a = 0.f;
#pragma unroll
    for (int w = 0; w < SD_WARPS; ++w) mm = fmaxf(mm, s_m[w][h]);
#pragma unroll
    for (int w = 0; w < SD_WARPS; ++w)
      a += s_m[w][h] == -INFINITY ? 0.f : s_o[((size_t)w * GH + h) * dv + c] * expf(s_m[w][h] - mm);
    record(h)[2 + c] = a;
  }
  if (threadIdx.x < ng) {
    const int h = threadIdx.x;
    float mm = -INFINITY, ll = 0.f;
#pragma unroll
    for (int w = 0; w < SD_WARPS; ++w) mm = fmaxf(mm, s_m[w][h]);
#pragma unroll
    for (int w = 0; w < SD_WARPS; ++w) ll += s_m[w][h] == -INFINITY ? 0.f : s_l[w][h] * expf(s_m[w][h] - mm);
    float* pp = record(h);
    pp[0] = mm;
    pp[1] = ll;
  }
}

template <typename T>
__global__ void scored_decode_merge_kernel(const float* __restrict__ part, T* __restrict__ out, long long out_stride,
                                           const int* __restrict__ dec_reqs, const int* __restrict__ q_start,
                                           int max_splits, int n_q_heads, int dv, const float* __restrict__ sink,
                                           float out_scale) {
  const int di = blockIdx.x, head = blockIdx.y;
  const float* base = part + ((size_t)di * n_q_heads + head) * max_splits * sd_part_stride(dv);
  float m = sink ? sink[head] : -INFINITY;
  for (int s = 0; s < max_splits; ++s) m = fmaxf(m, base[(size_t)s * sd_part_stride(dv)]);
  float l = sink ? expf(sink[head] - m) : 0.f;
  for (int s = 0; s < max_splits; ++s) {
    const float* pp = base + (size_t)s * sd_part_stride(dv);
    if (pp[0] > -INFINITY) l += pp[1] * expf(pp[0] - m);
  }
  const float inv = l > 0.f ? out_scale / l : 0.f;
  T* o = out + (size_t)q_start[dec_reqs[di]] * out_stride + (size_t)head * dv;
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < max_splits; ++s) {
      const float* pp = base + (size_t)s * sd_part_stride(dv);
      if (pp[0] > -INFINITY) a += pp[2 + c] * expf(pp[0] - m);
    }
    o[c] = from_float<T>(a * inv);
  }
}

// How many query heads of a key head one block of the decode kernel takes (1, 2 or 4), or 0 where rows cannot be read
// sixteen bytes a load (key rows of a whole number of such loads, value rows of a multiple of four channels) and the
// kernel of a block per query head runs. Callers size a step's runs of keys by it.
LLMRS_API int llmrs_scored_decode_group(int n_q_heads, int n_kv_heads, int dk, int dv, int page_size, int dtype) {
  const int cw = dtype == LLMRS_F32 ? 4 : 8;
  if (n_kv_heads <= 0 || n_q_heads % n_kv_heads || dk % cw || dv % 4 || dk > 32 * SD_MAXC || dv > 32 * SD_MAXC ||
      ((long long)page_size * (dk + dv)) % cw)
    return 0;
  const int G = n_q_heads / n_kv_heads;
  return G >= 3 ? 4 : G;
}

LLMRS_API long long llmrs_scored_decode_scratch_floats(int n_dec, int n_q_heads, int dv, int max_splits) {
  return (long long)n_dec * n_q_heads * max_splits * (long long)sd_part_stride(dv);
}

// `max_splits` runs of `split_keys` keys, counted from each request's first visible key, must cover the longest
// visible span; scratch holds llmrs_scored_decode_scratch_floats floats.
LLMRS_API int llmrs_scored_decode(const void* q, long long q_stride, void* out, long long out_stride,
                                  const void* cache, const int* dec_reqs, int n_dec, const int* q_start,
                                  const int* cached_len, const int* block_table, int table_stride, float* scratch,
                                  int max_splits, int split_keys, int n_q_heads, int n_kv_heads, int dk, int dv,
                                  int page_size, float scale, float softcap, const float* sink, int mask,
                                  int mask_size, const float* bias, int bias_len, float out_scale, int dtype,
                                  cudaStream_t stream) {
  LLMRS_REQUIRE(n_dec >= 0 && n_q_heads > 0 && n_kv_heads > 0 && page_size > 0 && max_splits > 0 && split_keys > 0,
                "scored_decode: bad sizes");
  LLMRS_REQUIRE(n_q_heads % n_kv_heads == 0, "scored_decode: %d query heads are no multiple of %d key heads",
                n_q_heads, n_kv_heads);
  LLMRS_REQUIRE(dk >= 1 && dk <= 32 * SD_MAXC && dv >= 1 && dv <= 32 * SD_MAXC, "scored_decode: head sizes %d / %d", dk, dv);
  LLMRS_REQUIRE(mask == MASK_CAUSAL || ((mask == MASK_WINDOW || mask == MASK_CHUNK) && mask_size > 0),
                "scored_decode: mask %d with size %d", mask, mask_size);
  LLMRS_REQUIRE(n_q_heads <= 65535 && max_splits <= 65535, "scored_decode: too many heads or runs");
  LLMRS_REQUIRE(bias == nullptr || bias_len > 0, "scored_decode: a bias table of %d rows", bias_len);
  if (n_dec == 0) return 0;
  ScoreOpts opt{scale, softcap, sink, mask, mask_size, bias, bias_len, n_q_heads, out_scale};
  dim3 grid(n_dec, n_q_heads, max_splits), mgrid(n_dec, n_q_heads);
  const size_t smem = (size_t)SD_WARPS * dv * sizeof(float);
  // Rows of a multiple of four channels that start on a load's boundary are read four channels a load.
  const size_t esz = dtype == LLMRS_F32 ? 4 : 2;
  const bool vec = dk % 4 == 0 && dv % 4 == 0 && ((uintptr_t)q % (4 * esz)) == 0 && q_stride % 4 == 0 &&
                   ((uintptr_t)cache % (4 * esz)) == 0;
  const int gh = llmrs_scored_decode_group(n_q_heads, n_kv_heads, dk, dv, page_size, dtype);
  const bool grouped = gh > 0 && ((uintptr_t)cache & 15) == 0 && !g_scored_generic_only;
  const int G = n_q_heads / n_kv_heads;
  dim3 ggrid(n_dec, grouped ? n_kv_heads * ((G + gh - 1) / gh) : 1, max_splits);
  const size_t gsmem = grouped ? ((size_t)gh * dk + (size_t)SD_WARPS * gh * dv) * sizeof(float) : 0;
  LLMRS_REQUIRE(ggrid.y <= 65535, "scored_decode: too many head groups");
#define LLMRS_SG_LAUNCH(T, GH, VG)                                                                                    \
  scored_decode_grouped_kernel<T, GH, VG><<<ggrid, SD_THREADS, gsmem, stream>>>(                                      \
      (const T*)q, q_stride, (const T*)cache, dec_reqs, q_start, cached_len, block_table, table_stride, scratch,      \
      max_splits, split_keys, n_q_heads, n_kv_heads, dk, dv, page_size, opt)
#define LLMRS_SD_LAUNCH(T)                                                                                            \
  do {                                                                                                                \
    if (grouped) {                                                                                                    \
      if (dv <= 128) {                                                                                                \
        if (gh == 1) LLMRS_SG_LAUNCH(T, 1, 1);                                                                        \
        else if (gh == 2) LLMRS_SG_LAUNCH(T, 2, 1);                                                                   \
        else LLMRS_SG_LAUNCH(T, 4, 1);                                                                                \
      } else {                                                                                                        \
        if (gh == 1) LLMRS_SG_LAUNCH(T, 1, 2);                                                                        \
        else if (gh == 2) LLMRS_SG_LAUNCH(T, 2, 2);                                                                   \
        else LLMRS_SG_LAUNCH(T, 4, 2);                                                                                \
      }                                                                                                               \
    } else if (vec)                                                                                                   \
      scored_decode_kernel<T, true><<<grid, SD_THREADS, smem, stream>>>(                                              \
          (const T*)q, q_stride, (const T*)cache, dec_reqs, q_start, cached_len, block_table, table_stride, scratch,  \
          max_splits, split_keys, n_q_heads, n_kv_heads, dk, dv, page_size, opt);                                     \
    else                                                                                                              \
      scored_decode_kernel<T, false><<<grid, SD_THREADS, smem, stream>>>(                                             \
          (const T*)q, q_stride, (const T*)cache, dec_reqs, q_start, cached_len, block_table, table_stride, scratch,  \
          max_splits, split_keys, n_q_heads, n_kv_heads, dk, dv, page_size, opt);                                     \
  } while (0)
  if (dtype == LLMRS_F32) {
    LLMRS_SD_LAUNCH(float);
    int rc = llmrs_launch_status("scored_decode");
    if (rc) return rc;
    scored_decode_merge_kernel<float><<<mgrid, 64, 0, stream>>>(scratch, (float*)out, out_stride, dec_reqs, q_start,
                                                                max_splits, n_q_heads, dv, sink, out_scale);
  } else if (dtype == LLMRS_BF16) {
    LLMRS_SD_LAUNCH(bf16);
    int rc = llmrs_launch_status("scored_decode");
    if (rc) return rc;
    scored_decode_merge_kernel<bf16><<<mgrid, 64, 0, stream>>>(scratch, (bf16*)out, out_stride, dec_reqs, q_start,
                                                               max_splits, n_q_heads, dv, sink, out_scale);
  } else {
    return llmrs_fail("scored_decode: unknown dtype %d", dtype);
  }
#undef LLMRS_SD_LAUNCH
#undef LLMRS_SG_LAUNCH
  return llmrs_launch_status("scored_decode (merge)");
}
