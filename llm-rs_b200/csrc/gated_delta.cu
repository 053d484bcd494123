// Gated delta rule: a recurrent mixer with a matrix state S [key channel, value channel] per head,
//
//   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (the read-out sees the token's own write)
//
// g in (0, 1) and beta in (0, 1) are one number per head and token. q and k (G heads of d channels; value head h reads
// q/k head h / (H / G)) and v (H heads of dv channels) each pass a short causal convolution over time per channel
// (K taps, the last one the current token's, zeros before a sequence's start) and SiLU; q and k are then made unit
// vectors per head (x / sqrt(sum x^2 + key_eps)), q is also multiplied by q_scale. g = exp(-exp(A_log_h) *
// softplus(a + dt_bias_h)) and beta = sigmoid(b) come from two float32 projections a, b. After the recurrence each head's
// o is divided by its root mean square over dv, multiplied by a weight of size dv (shared by the heads) and by
// SiLU(gate). Everything but the projections' inputs is float32.
//
// Per-request state: S (float32 [slots, H, d, dv]) and the last K - 1 rows that entered the convolutions
// (float32 [slots, K - 1, C], C = 2 G d + H dv: the q, k and v channels side by side, oldest row first).
//
//   prepare      a block per token: convolutions + SiLU, unit q and k, g and beta, as float32 rows
//   conv state   a block per request, after prepare: the request's last K - 1 convolution inputs
//   recurrence   a block per (request, head, slice of 16 value columns) walks the request's tokens in order; four
//                neighbouring lanes share a column, each with a quarter of the key channels in registers (lane p of the
//                four holds channels 4 (p + 4 j) .. 4 (p + 4 j) + 3, so that the four read neighbouring 16-byte pieces
//                of a row in shared memory, not pieces a bank's stride apart); k^T S and q^T S are summed over the four
//                by two shuffles. Rows come in chunks through two shared-memory buffers.
//   output       a warp per (token, head): norm, weight, gate
//
// Long portions take the recurrence in CHUNKS of 32 tokens instead (the same numbers up to float32 rounding, all of it
// float32 FMA). Within a chunk that starts from the state S_0, with L_t the sum of log g up to and including token t:
//
//   u_t = beta_t (v_t - e^{L_t} S_0^T k_t - sum_{s<t} A[t,s] u_s),     A[t,s] = e^{L_t - L_s} (k_t . k_s)
//   =>  U = T (V - diag(e^L) K S_0),   T = (I + diag(beta) A)^{-1} diag(beta)      (32 x 32, lower triangular)
//   o_t = e^{L_t} S_0^T q_t + sum_{s<=t} P[t,s] u_s,                    P[t,s] = e^{L_t - L_s} (q_t . k_s)
//   S_32 = e^{L_32} S_0 + K^T diag(e^{L_32 - L_s}) U
//
// T, P and the decays depend on no state: `chunk tables` makes them for every chunk and head at once (a block each).
// `chunked recurrence` then walks a request's chunks with a block per (request, head, 16 value columns): five small
// products per chunk over rows that arrive through two shared-memory buffers, 32 tokens per sequential step instead of
// one. A chunk's missing tokens (a portion's end) count as k = q = v = 0, beta = 0, g = 1 and change nothing.
// The chunked form is OFF by default (llmrs_gated_delta_chunked): its products read every operand from shared memory
// and are bound by that, so it does not beat the walk yet.
#include "common.cuh"
#include "mma_util.cuh"

__device__ __forceinline__ float gd_silu(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float gd_softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

template <typename TA>
__global__ void gdr_prepare_kernel(const TA* __restrict__ x, long long stride, const float* __restrict__ taps,
                                   const float* __restrict__ ba, const float* __restrict__ a_log,
                                   const float* __restrict__ dt_bias, const float* __restrict__ conv_state,
                                   const int* __restrict__ token_req, const int* __restrict__ q_start,
                                   const int* __restrict__ slot_ids, float* __restrict__ pq, float* __restrict__ pk,
                                   float* __restrict__ pv, float* __restrict__ pbeta, float* __restrict__ pg,
                                   float* __restrict__ plg, int G, int H, int d, int dv, int K, float key_eps,
                                   float q_scale) {
  extern __shared__ float row[];      // [C] after convolution and SiLU
  const int t = blockIdx.x, req = token_req[t], off = t - q_start[req];
  const int wq = G * d, wv = H * dv, C = 2 * wq + wv;
  const float* tail = conv_state + (size_t)slot_ids[req] * (K - 1) * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < K; ++j) {      // lag j: the input of j tokens ago
      const int o = off - j;
      const float in = o >= 0 ? to_float(x[(size_t)(t - j) * stride + c]) : tail[(size_t)(K - 1 + o) * C + c];
      acc = fmaf(taps[(size_t)c * K + (K - 1 - j)], in, acc);
    }
    row[c] = gd_silu(acc);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int hh = warp; hh < 2 * G; hh += nwarps) {      // q heads, then k heads
    const float* src = row + (size_t)hh * d;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) ss = fmaf(src[i], src[i], ss);
    const float inv = 1.0f / sqrtf(warp_sum(ss) + key_eps) * (hh < G ? q_scale : 1.0f);
    float* dst = hh < G ? pq + (size_t)t * wq + (size_t)hh * d : pk + (size_t)t * wq + (size_t)(hh - G) * d;
    for (int i = lane; i < d; i += 32) dst[i] = src[i] * inv;
  }
  for (int c = threadIdx.x; c < wv; c += blockDim.x) pv[(size_t)t * wv + c] = row[2 * wq + c];
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    pbeta[(size_t)t * H + h] = 1.0f / (1.0f + expf(-ba[(size_t)t * 2 * H + h]));
    const float lg = -expf(a_log[h]) * gd_softplus(ba[(size_t)t * 2 * H + H + h] + dt_bias[h]);      // log g
    plg[(size_t)t * H + h] = lg;
    pg[(size_t)t * H + h] = expf(lg);
  }
}

template <typename TA>
__global__ void gdr_conv_state_kernel(const TA* __restrict__ x, long long stride, float* __restrict__ conv_state,
                                      const int* __restrict__ q_start, const int* __restrict__ n_new,
                                      const int* __restrict__ slot_ids, int C, int K) {
  const int req = blockIdx.x, n = n_new[req], t0 = q_start[req];
  float* tail = conv_state + (size_t)slot_ids[req] * (K - 1) * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x)
    for (int j = 0; j < K - 1; ++j) {      // ascending: an old row is read before the place it moves from is overwritten
      const int o = n - (K - 1) + j;
      tail[(size_t)j * C + c] = o >= 0 ? to_float(x[(size_t)(t0 + o) * stride + c]) : tail[(size_t)(j + n) * C + c];
    }
}

constexpr int GD_COLS = 16;      // value columns of a block
#ifndef LLMRS_GD_LANES
#define LLMRS_GD_LANES 8
#endif

// LANES: neighbouring lanes that share a column (4, 8 or 16; at most DMAX / 4, so that a lane holds whole pieces of
// four channels).
template <int DMAX, int LANES>
__global__ void __launch_bounds__(GD_COLS * LANES)
gdr_recurrence_kernel(const float* __restrict__ pq, const float* __restrict__ pk, const float* __restrict__ pv,
                      const float* __restrict__ pbeta, const float* __restrict__ pg, float* __restrict__ state,
                      const int* __restrict__ q_start, const int* __restrict__ n_new,
                      const int* __restrict__ slot_ids, float* __restrict__ o_raw, int G, int H, int d, int dv) {
  constexpr int CHUNK = DMAX >= 256 ? 8 : 16;
  constexpr int GD_LANES = LANES, GD_THREADS = GD_COLS * LANES;
  constexpr int IPL = DMAX / GD_LANES;             // key channels per lane
  __shared__ __align__(16) float s_qk[2][2][CHUNK][DMAX];      // q, k of a chunk's tokens; channels >= d stay 0
  __shared__ float s_v[2][CHUNK][GD_COLS], s_bg[2][2][CHUNK];
  // The lanes' shares of a chunk's read-outs: summed over a column's lanes after the chunk's walk, by all threads at
  // once, instead of by a chain of shuffles in every token's turn (the walk then waits for one such chain a token,
  // the one it cannot do without: k^T S).
  __shared__ float s_o[CHUNK][GD_COLS][LANES + 1];
  const int req = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * GD_COLS;
  const int kh = head / (H / G);
  const int tid = threadIdx.x;
  const int col = col0 + tid / GD_LANES, part = tid % GD_LANES;
  // Register i of a lane holds key channel ch(i): pieces of four channels dealt out to the four lanes in turn.
  auto ch = [&](int i) { return ((i >> 2) * GD_LANES + part) * 4 + (i & 3); };
  const bool live = col < dv;
  const int t0 = q_start[req], n = n_new[req];
  const int wq = G * d, wv = H * dv;
  float* S_g = state + ((size_t)slot_ids[req] * H + head) * d * dv;
  float S[IPL];
#pragma unroll
  for (int i = 0; i < IPL; ++i) S[i] = (live && ch(i) < d) ? S_g[(size_t)ch(i) * dv + col] : 0.f;
  for (int e = tid; e < 2 * 2 * CHUNK * DMAX; e += GD_THREADS) (&s_qk[0][0][0][0])[e] = 0.f;
  for (int e = tid; e < 2 * CHUNK * GD_COLS; e += GD_THREADS) (&s_v[0][0][0])[e] = 0.f;
  __syncthreads();
  const bool wide = d % 4 == 0;      // every row then starts on a 16-byte boundary
  const int ncols = min(GD_COLS, dv - col0);
  auto load_chunk = [&](int buf, int c0) {
    const int cn = min(CHUNK, n - c0);
    if (wide) {
      const int per_row = d / 4;
      for (int e = tid; e < 2 * cn * per_row; e += GD_THREADS) {
        const int a = e / (cn * per_row), rem = e % (cn * per_row), tt = rem / per_row, piece = rem % per_row;
        const float* src = (a == 0 ? pq : pk) + (size_t)(t0 + c0 + tt) * wq + (size_t)kh * d + piece * 4;
        cp_async_16(&s_qk[buf][a][tt][piece * 4], src, 16);
      }
    } else {
      for (int e = tid; e < 2 * cn * d; e += GD_THREADS) {
        const int a = e / (cn * d), rem = e % (cn * d), tt = rem / d, i = rem % d;
        s_qk[buf][a][tt][i] = (a == 0 ? pq : pk)[(size_t)(t0 + c0 + tt) * wq + (size_t)kh * d + i];
      }
    }
    for (int e = tid; e < cn * ncols; e += GD_THREADS) {
      const int tt = e / ncols, c = e % ncols;
      s_v[buf][tt][c] = pv[(size_t)(t0 + c0 + tt) * wv + (size_t)head * dv + col0 + c];
    }
    for (int e = tid; e < 2 * cn; e += GD_THREADS) {
      const int a = e / cn, tt = e % cn;
      s_bg[buf][a][tt] = (a == 0 ? pbeta : pg)[(size_t)(t0 + c0 + tt) * H + head];
    }
    cp_async_commit();
  };

  if (n > 0) load_chunk(0, 0);
  for (int c0 = 0, it = 0; c0 < n; c0 += CHUNK, ++it) {
    const int cn = min(CHUNK, n - c0), buf = it & 1;
    if (c0 + CHUNK < n) {
      load_chunk(buf ^ 1, c0 + CHUNK);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
#pragma unroll 4
    for (int tt = 0; tt < cn; ++tt) {
      const float vj = s_v[buf][tt][tid / GD_LANES], beta = s_bg[buf][0][tt], g = s_bg[buf][1][tt];
      float ks[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < IPL; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(&s_qk[buf][1][tt][ch(i)]);
        S[i] *= g; S[i + 1] *= g; S[i + 2] *= g; S[i + 3] *= g;
        ks[0] = fmaf(k4.x, S[i], ks[0]);
        ks[1] = fmaf(k4.y, S[i + 1], ks[1]);
        ks[2] = fmaf(k4.z, S[i + 2], ks[2]);
        ks[3] = fmaf(k4.w, S[i + 3], ks[3]);
      }
      float kS = (ks[0] + ks[1]) + (ks[2] + ks[3]);
#pragma unroll
      for (int off = 1; off < LANES; off <<= 1) kS += __shfl_xor_sync(0xffffffffu, kS, off);
      const float u = beta * (vj - kS);
      float os[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < IPL; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(&s_qk[buf][1][tt][ch(i)]);
        const float4 q4 = *reinterpret_cast<const float4*>(&s_qk[buf][0][tt][ch(i)]);
        S[i] = fmaf(k4.x, u, S[i]);
        S[i + 1] = fmaf(k4.y, u, S[i + 1]);
        S[i + 2] = fmaf(k4.z, u, S[i + 2]);
        S[i + 3] = fmaf(k4.w, u, S[i + 3]);
        os[0] = fmaf(S[i], q4.x, os[0]);
        os[1] = fmaf(S[i + 1], q4.y, os[1]);
        os[2] = fmaf(S[i + 2], q4.z, os[2]);
        os[3] = fmaf(S[i + 3], q4.w, os[3]);
      }
      s_o[tt][tid / GD_LANES][part] = (os[0] + os[1]) + (os[2] + os[3]);
    }
    __syncthreads();
    for (int e = tid; e < cn * GD_COLS; e += GD_THREADS) {
      const int tt = e / GD_COLS, c = e % GD_COLS;
      float o = 0.f;
#pragma unroll
      for (int p = 0; p < LANES; ++p) o += s_o[tt][c][p];
      if (col0 + c < dv) o_raw[(size_t)(t0 + c0 + tt) * wv + (size_t)head * dv + col0 + c] = o;
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < IPL; ++i)
      if (ch(i) < d) S_g[(size_t)ch(i) * dv + col] = S[i];
  }
}


// ---- the recurrence in chunks ------------------------------------------------------------------------------------
constexpr int GC_C = 32, GC_W = 16, GC_THREADS = 128, GC_TST = GC_C + 4;
// A chunk's tables in the workspace: T [C][C], P [C][C], e^{L_t} [C], e^{L_C - L_t} [C].
constexpr int GC_TABLE = 2 * GC_C * GC_C + 2 * GC_C;
// The place of request `req`'s chunk `k`: requests' chunks follow one another; floor(q_start / C) + req leaves every
// request at least ceil(n / C) places.
__device__ __forceinline__ int gc_slot(int q_start, int req, int k) { return q_start / GC_C + req + k; }

__global__ void __launch_bounds__(GC_THREADS)
gdr_chunk_tables_kernel(const float* __restrict__ pq, const float* __restrict__ pk, const float* __restrict__ pbeta,
                        const float* __restrict__ plg, const int* __restrict__ q_start, const int* __restrict__ n_new,
                        float* __restrict__ tables, int G, int H, int d) {
  extern __shared__ float sm[];
  const int req = blockIdx.x, chunk = blockIdx.y, head = blockIdx.z;
  const int n = n_new[req], c0 = chunk * GC_C;
  if (c0 >= n) return;
  const int cn = min(GC_C, n - c0), t0 = q_start[req] + c0, kh = head / (H / G), wq = G * d, st = d + 1;
  float* Ks = sm;                      // [C][d + 1]
  float* Qs = Ks + GC_C * st;          // [C][d + 1]
  float* A = Qs + GC_C * st;           // [C][C + 1]
  float* L = A + GC_C * (GC_C + 1);    // [C]
  float* B = L + GC_C;                 // [C]
  float* out = tables + ((size_t)gc_slot(q_start[req], req, chunk) * H + head) * GC_TABLE;
  for (int e = threadIdx.x; e < GC_C * d; e += GC_THREADS) {
    const int t = e / d, i = e % d;
    Ks[t * st + i] = t < cn ? pk[(size_t)(t0 + t) * wq + (size_t)kh * d + i] : 0.f;
    Qs[t * st + i] = t < cn ? pq[(size_t)(t0 + t) * wq + (size_t)kh * d + i] : 0.f;
  }
  if (threadIdx.x < GC_C) B[threadIdx.x] = threadIdx.x < cn ? pbeta[(size_t)(t0 + threadIdx.x) * H + head] : 0.f;
  if (threadIdx.x == 0) {
    float run = 0.f;
    for (int t = 0; t < GC_C; ++t) {
      if (t < cn) run += plg[(size_t)(t0 + t) * H + head];
      L[t] = run;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < GC_C * GC_C; e += GC_THREADS) {
    const int t = e / GC_C, s_ = e % GC_C;
    float a = 0.f, p = 0.f;
    if (s_ <= t) {
      const float* kt = Ks + t * st;
      const float* qt = Qs + t * st;
      const float* ks = Ks + s_ * st;
      for (int i = 0; i < d; ++i) {
        a = fmaf(kt[i], ks[i], a);
        p = fmaf(qt[i], ks[i], p);
      }
      const float w = expf(L[t] - L[s_]);
      a *= w;
      p *= w;
    }
    A[t * (GC_C + 1) + s_] = s_ < t ? a : 0.f;
    out[GC_C * GC_C + e] = p;
  }
  if (threadIdx.x < GC_C) {
    out[2 * GC_C * GC_C + threadIdx.x] = expf(L[threadIdx.x]);
    out[2 * GC_C * GC_C + GC_C + threadIdx.x] = expf(L[GC_C - 1] - L[threadIdx.x]);
  }
  __syncthreads();
  // T = (I + diag(beta) A)^{-1} diag(beta) by forward substitution: a thread per column.
  if (threadIdx.x < GC_C) {
    const int c = threadIdx.x;
    float col[GC_C];
#pragma unroll
    for (int t = 0; t < GC_C; ++t) {
      float acc = t == c ? 1.0f : 0.f;
#pragma unroll
      for (int s_ = 0; s_ < GC_C; ++s_)
        if (s_ < t) acc = fmaf(-A[t * (GC_C + 1) + s_], col[s_], acc);
      col[t] = t >= c ? B[t] * acc : 0.f;
    }
#pragma unroll
    for (int t = 0; t < GC_C; ++t) out[t * GC_C + c] = col[t];
  }
}

// Shared memory of the chunked recurrence, in floats: two buffers of (K, Q rows [C][d + 4], T, P [C][C + 4], V [C][W],
// e^L, e^{L_C - L}), then the state slice [d][W], V' and U [C][W] each.
__host__ __device__ inline int gc_buffer_floats(int d) { return 2 * GC_C * (d + 4) + 2 * GC_C * GC_TST + GC_C * GC_W + 2 * GC_C; }
__host__ __device__ inline int gc_smem_floats(int d) { return 2 * gc_buffer_floats(d) + d * GC_W + 2 * GC_C * GC_W; }

__global__ void __launch_bounds__(GC_THREADS)
gdr_chunked_kernel(const float* __restrict__ pq, const float* __restrict__ pk, const float* __restrict__ pv,
                   const float* __restrict__ tables, float* __restrict__ state, const int* __restrict__ q_start,
                   const int* __restrict__ n_new, const int* __restrict__ slot_ids, float* __restrict__ o_raw, int G,
                   int H, int d, int dv) {
  extern __shared__ __align__(16) float sm[];
  const int req = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * GC_W;
  const int kh = head / (H / G), tid = threadIdx.x, j = tid & 15, grp = tid >> 4;      // 8 groups of 16 columns' lanes
  const int t_first = q_start[req], n = n_new[req], wq = G * d, wv = H * dv, kst = d + 4;
  const int ncols = min(GC_W, dv - col0);
  const int bufsz = gc_buffer_floats(d);
  float* S0 = sm + 2 * bufsz;            // [d][W]
  float* Vp = S0 + d * GC_W;             // [C][W]
  float* Us = Vp + GC_C * GC_W;          // [C][W]
  float* S_g = state + ((size_t)slot_ids[req] * H + head) * d * dv;
  for (int e = tid; e < d * GC_W; e += GC_THREADS) {
    const int i = e / GC_W, c = e % GC_W;
    S0[e] = c < ncols ? S_g[(size_t)i * dv + col0 + c] : 0.f;
  }
  const int n_chunks = (n + GC_C - 1) / GC_C;
  auto load = [&](int it) {
    float* b = sm + (it & 1) * bufsz;
    float* Ks = b;
    float* Qs = Ks + GC_C * kst;
    float* Ts = Qs + GC_C * kst;
    float* Ps = Ts + GC_C * GC_TST;
    float* Vs = Ps + GC_C * GC_TST;
    float* Gs = Vs + GC_C * GC_W;        // e^L [C], then e^{L_C - L} [C]
    const int c0 = it * GC_C, cn = min(GC_C, n - c0), per_row = d / 4;
    for (int e = tid; e < 2 * GC_C * per_row; e += GC_THREADS) {
      const int a = e / (GC_C * per_row), rem = e % (GC_C * per_row), t = rem / per_row, piece = rem % per_row;
      const bool valid = t < cn;
      const float* src = (a == 0 ? pk : pq) + (valid ? (size_t)(t_first + c0 + t) * wq + (size_t)kh * d + piece * 4 : 0);
      cp_async_16((a == 0 ? Ks : Qs) + t * kst + piece * 4, src, valid ? 16 : 0);
    }
    const float* tb = tables + ((size_t)gc_slot(t_first, req, it) * H + head) * GC_TABLE;
    for (int e = tid; e < 2 * GC_C * (GC_C / 4); e += GC_THREADS) {
      const int a = e / (GC_C * (GC_C / 4)), rem = e % (GC_C * (GC_C / 4)), t = rem / (GC_C / 4), piece = rem % (GC_C / 4);
      cp_async_16((a == 0 ? Ts : Ps) + t * GC_TST + piece * 4, tb + a * GC_C * GC_C + t * GC_C + piece * 4, 16);
    }
    for (int e = tid; e < GC_C * (GC_W / 4); e += GC_THREADS) {
      const int t = e / (GC_W / 4), piece = e % (GC_W / 4);
      const bool valid = t < cn && piece * 4 < ncols;      // dv is a multiple of 4: a piece lies wholly inside or outside
      const float* src = pv + (valid ? (size_t)(t_first + c0 + t) * wv + (size_t)head * dv + col0 + piece * 4 : 0);
      cp_async_16(Vs + t * GC_W + piece * 4, src, valid ? 16 : 0);
    }
    for (int e = tid; e < 2 * GC_C / 4; e += GC_THREADS) cp_async_16(Gs + e * 4, tb + 2 * GC_C * GC_C + e * 4, 16);
    cp_async_commit();
  };
  if (n_chunks > 0) load(0);
  for (int it = 0; it < n_chunks; ++it) {
    if (it + 1 < n_chunks) {
      load(it + 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const float* b = sm + (it & 1) * bufsz;
    const float* Ks = b;
    const float* Qs = Ks + GC_C * kst;
    const float* Ts = Qs + GC_C * kst;
    const float* Ps = Ts + GC_C * GC_TST;
    const float* Vs = Ps + GC_C * GC_TST;
    const float* Gs = Vs + GC_C * GC_W;
    const float* Ds = Gs + GC_C;
    const int c0 = it * GC_C, cn = min(GC_C, n - c0);
    // This thread's four tokens grp, grp + 8, grp + 16, grp + 24 of column j.
    float x[4] = {0.f, 0.f, 0.f, 0.f}, qs[4] = {0.f, 0.f, 0.f, 0.f};
    for (int i = 0; i < d; i += 4) {
      const float s0 = S0[(i + 0) * GC_W + j], s1 = S0[(i + 1) * GC_W + j], s2 = S0[(i + 2) * GC_W + j],
                  s3 = S0[(i + 3) * GC_W + j];
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        const float4 k4 = *reinterpret_cast<const float4*>(Ks + (grp + 8 * m) * kst + i);
        const float4 q4 = *reinterpret_cast<const float4*>(Qs + (grp + 8 * m) * kst + i);
        x[m] = fmaf(k4.w, s3, fmaf(k4.z, s2, fmaf(k4.y, s1, fmaf(k4.x, s0, x[m]))));
        qs[m] = fmaf(q4.w, s3, fmaf(q4.z, s2, fmaf(q4.y, s1, fmaf(q4.x, s0, qs[m]))));
      }
    }
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const int t = grp + 8 * m;
      Vp[t * GC_W + j] = Vs[t * GC_W + j] - Gs[t] * x[m];      // V - e^L (K S_0)
    }
    __syncthreads();
    float u[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s_ = 0; s_ < GC_C; s_ += 4) {
      const float v0 = Vp[(s_ + 0) * GC_W + j], v1 = Vp[(s_ + 1) * GC_W + j], v2 = Vp[(s_ + 2) * GC_W + j],
                  v3 = Vp[(s_ + 3) * GC_W + j];
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        const float4 t4 = *reinterpret_cast<const float4*>(Ts + (grp + 8 * m) * GC_TST + s_);
        u[m] = fmaf(t4.w, v3, fmaf(t4.z, v2, fmaf(t4.y, v1, fmaf(t4.x, v0, u[m]))));
      }
    }
#pragma unroll
    for (int m = 0; m < 4; ++m) Us[(grp + 8 * m) * GC_W + j] = u[m];
    __syncthreads();
    float o[4];
#pragma unroll
    for (int m = 0; m < 4; ++m) o[m] = Gs[grp + 8 * m] * qs[m];
    for (int s_ = 0; s_ < GC_C; s_ += 4) {
      const float u0 = Us[(s_ + 0) * GC_W + j], u1 = Us[(s_ + 1) * GC_W + j], u2 = Us[(s_ + 2) * GC_W + j],
                  u3 = Us[(s_ + 3) * GC_W + j];
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        const float4 p4 = *reinterpret_cast<const float4*>(Ps + (grp + 8 * m) * GC_TST + s_);
        o[m] = fmaf(p4.w, u3, fmaf(p4.z, u2, fmaf(p4.y, u1, fmaf(p4.x, u0, o[m]))));
      }
    }
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const int t = grp + 8 * m;
      if (t < cn && j < ncols) o_raw[(size_t)(t_first + c0 + t) * wv + (size_t)head * dv + col0 + j] = o[m];
    }
    // The new state: this thread's key channels [i_lo, i_hi) of column j.
    const int per = ((d + 7) / 8 + 3) & ~3, i_lo = min(grp * per, d), i_hi = min(i_lo + per, d);
    float acc[32];
#pragma unroll
    for (int a = 0; a < 32; ++a) acc[a] = 0.f;
    for (int t = 0; t < GC_C; ++t) {
      const float du = Ds[t] * Us[t * GC_W + j];
#pragma unroll
      for (int a = 0; a < 32; a += 4) {
        if (i_lo + a < i_hi) {
          const float4 k4 = *reinterpret_cast<const float4*>(Ks + t * kst + i_lo + a);
          acc[a] = fmaf(k4.x, du, acc[a]);
          acc[a + 1] = fmaf(k4.y, du, acc[a + 1]);
          acc[a + 2] = fmaf(k4.z, du, acc[a + 2]);
          acc[a + 3] = fmaf(k4.w, du, acc[a + 3]);
        }
      }
    }
    __syncthreads();      // every thread has read the old state
    const float gc = Gs[GC_C - 1];
#pragma unroll
    for (int a = 0; a < 32; ++a)
      if (i_lo + a < i_hi) S0[(i_lo + a) * GC_W + j] = fmaf(gc, S0[(i_lo + a) * GC_W + j], acc[a]);
    // (the next turn's first barrier makes the new state visible; its loads go into the other buffer)
  }
  __syncthreads();
  for (int e = tid; e < d * GC_W; e += GC_THREADS) {
    const int i = e / GC_W, c = e % GC_W;
    if (c < ncols) S_g[(size_t)i * dv + col0 + c] = S0[e];
  }
}

// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * weight[:] * silu(gate[t, h, :]); a warp per (t, h).
template <typename TA>
__global__ void gdr_out_kernel(const float* __restrict__ o_raw, const TA* __restrict__ gate, long long gate_stride,
                               const float* __restrict__ norm_w, TA* __restrict__ out, long long out_stride,
                               int n_rows, int H, int dv, float eps, float out_scale) {
  const int r = blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= n_rows) return;
  const int t = r / H, h = r % H;
  const float* o = o_raw + (size_t)t * H * dv + (size_t)h * dv;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) ss = fmaf(o[i], o[i], ss);
  const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps) * out_scale;
  for (int i = lane; i < dv; i += 32) {
    const float gt = gd_silu(to_float(gate[(size_t)t * gate_stride + (size_t)h * dv + i]));
    out[(size_t)t * out_stride + (size_t)h * dv + i] = from_float<TA>(o[i] * inv * norm_w[i] * gt);
  }
}

static int launch_chunked(const float* pq, const float* pk, const float* pv, const float* pbeta, const float* plg,
                          float* tables, float* state, const int* q_start, const int* n_new, const int* slot_ids,
                          float* o_raw, int n_requests, int max_chunks, int G, int H, int d, int dv,
                          cudaStream_t stream) {
  const size_t smem_t = ((size_t)2 * GC_C * (d + 1) + GC_C * (GC_C + 1) + 2 * GC_C) * sizeof(float);
  const size_t smem_c = (size_t)gc_smem_floats(d) * sizeof(float);
  static size_t configured_t = 48 * 1024, configured_c = 48 * 1024;
  if (smem_t > configured_t) {
    cudaError_t e = cudaFuncSetAttribute(gdr_chunk_tables_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_t);
    if (e != cudaSuccess) return llmrs_fail("gated_delta: shared memory %zu: %s", smem_t, cudaGetErrorString(e));
    configured_t = smem_t;
  }
  if (smem_c > configured_c) {
    cudaError_t e = cudaFuncSetAttribute(gdr_chunked_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_c);
    if (e != cudaSuccess) return llmrs_fail("gated_delta: shared memory %zu: %s", smem_c, cudaGetErrorString(e));
    configured_c = smem_c;
  }
  LLMRS_REQUIRE(max_chunks <= 65535, "gated_delta: a portion of %d chunks is too long", max_chunks);
  gdr_chunk_tables_kernel<<<dim3(n_requests, max_chunks, H), GC_THREADS, smem_t, stream>>>(pq, pk, pbeta, plg, q_start,
                                                                                           n_new, tables, G, H, d);
  int rc = llmrs_launch_status("gated_delta (chunk tables)");
  if (rc != 0) return rc;
  gdr_chunked_kernel<<<dim3(n_requests, H, (dv + GC_W - 1) / GC_W), GC_THREADS, smem_c, stream>>>(
      pq, pk, pv, tables, state, q_start, n_new, slot_ids, o_raw, G, H, d, dv);
  return llmrs_launch_status("gated_delta (chunked recurrence)");
}

// Float32 workspace of the kernels, in floats: prepared q, k, v, beta, g and the raw read-outs.
LLMRS_API long long llmrs_gated_delta_work_floats(int n_tokens, int n_requests, int G, int H, int d, int dv) {
  const long long chunk_places = n_tokens / GC_C + n_requests + 1;
  return (long long)n_tokens * (2LL * G * d + 2LL * H * dv + 3LL * H) + 24 + chunk_places * H * GC_TABLE;
}

static int g_gd_chunked = 0;
// 1: portions of 64 tokens and more take the chunked form (off by default: it is not ahead yet, see the file's head).
LLMRS_API void llmrs_gated_delta_chunked(int on) { g_gd_chunked = on; }

// x: [tokens, >= 2 G d + H dv] of `dtype`, rows `x_stride` apart: the q, k and v channels that enter the convolutions;
// gate: [tokens, H dv] rows `gate_stride` apart; taps: float32 [2 G d + H dv, K]; ba: float32 [tokens, 2 H] (b, then
// a); state: float32 [slots, H, d, dv]; conv_state: float32 [slots, K - 1, 2 G d + H dv]; work: 16-byte aligned;
// out: [tokens, H dv] rows `out_stride` apart, multiplied by `out_scale`.
LLMRS_API int llmrs_gated_delta(const void* x, long long x_stride, const void* gate, long long gate_stride, int dtype,
                                const float* taps, const float* ba, const float* a_log, const float* dt_bias,
                                const float* norm_w, float* state, float* conv_state, const int* token_req,
                                const int* q_start, const int* n_new, const int* slot_ids, float* work, void* out,
                                long long out_stride, int n_tokens, int n_requests, int G, int H, int d, int dv, int K,
                                float key_eps, float q_scale, float norm_eps, float out_scale, cudaStream_t stream) {
  LLMRS_REQUIRE(n_requests >= 0 && n_tokens >= 0 && G > 0 && H > 0 && d > 0 && dv > 0 && K >= 1, "gated_delta: bad sizes");
  LLMRS_REQUIRE(H % G == 0, "gated_delta: %d value heads are no multiple of %d key heads", H, G);
  LLMRS_REQUIRE(d <= 256, "gated_delta: key heads of at most 256 channels, got %d", d);
  LLMRS_REQUIRE(H <= 65535 && (dv + GD_COLS - 1) / GD_COLS <= 65535, "gated_delta: too many heads or columns");
  LLMRS_REQUIRE(((uintptr_t)work & 15) == 0, "gated_delta: the workspace must be 16-byte aligned");
  if (n_requests == 0 || n_tokens == 0) return 0;
  const int wq = G * d, wv = H * dv, C = 2 * wq + wv;
  LLMRS_REQUIRE((size_t)C * sizeof(float) <= 160 * 1024, "gated_delta: %d convolution channels are too many", C);
  // Every piece starts on a 16-byte boundary (the recurrence copies q and k rows sixteen bytes at a time).
  auto up4 = [](size_t v) { return (v + 3) & ~(size_t)3; };
  float* pq = work;
  float* pk = pq + up4((size_t)n_tokens * wq);
  float* pv = pk + up4((size_t)n_tokens * wq);
  float* pbeta = pv + up4((size_t)n_tokens * wv);
  float* pg = pbeta + up4((size_t)n_tokens * H);
  float* plg = pg + up4((size_t)n_tokens * H);
  float* o_raw = plg + up4((size_t)n_tokens * H);
  float* tables = o_raw + up4((size_t)n_tokens * wv);
  // The chunked form where some request may bring 64 tokens or more (what the host knows: tokens and requests) and the
  // rows can be copied sixteen bytes at a time.
  const bool chunked = g_gd_chunked && n_tokens - n_requests + 1 >= 2 * GC_C && d % 4 == 0 && dv % 4 == 0 &&
                       (size_t)gc_smem_floats(d) * sizeof(float) <= 200 * 1024;
  const int max_chunks = (n_tokens - n_requests + 1 + GC_C - 1) / GC_C;
  const size_t smem = (size_t)C * sizeof(float);
  const int dmax = d <= 32 ? 32 : (d <= 64 ? 64 : (d <= 128 ? 128 : 256));
  dim3 grid(n_requests, H, (dv + GD_COLS - 1) / GD_COLS);
  const int rows = n_tokens * H;
#define LLMRS_GD_REC(DMAX, LANES)                                                                                 \
  gdr_recurrence_kernel<DMAX, LANES><<<grid, GD_COLS * LANES, 0, stream>>>(pq, pk, pv, pbeta, pg, state, q_start, n_new, \
                                                                           slot_ids, o_raw, G, H, d, dv)
#define LLMRS_GD_LAUNCH(T)                                                                                             \
  do {                                                                                                                 \
    static size_t configured = 48 * 1024;                                                                              \
    if (smem > configured) {                                                                                           \
      cudaError_t e = cudaFuncSetAttribute(gdr_prepare_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return llmrs_fail("gated_delta: shared memory %zu: %s", smem, cudaGetErrorString(e));      \
      configured = smem;                                                                                               \
    }                                                                                                                  \
    gdr_prepare_kernel<T><<<n_tokens, 256, smem, stream>>>((const T*)x, x_stride, taps, ba, a_log, dt_bias, conv_state, \
                                                           token_req, q_start, slot_ids, pq, pk, pv, pbeta, pg, plg,   \
                                                           G, H, d, dv, K, key_eps, q_scale);                          \
    int rc = llmrs_launch_status("gated_delta (prepare)");                                                             \
    if (rc != 0) return rc;                                                                                            \
    if (K > 1) {                                                                                                       \
      gdr_conv_state_kernel<T><<<n_requests, 256, 0, stream>>>((const T*)x, x_stride, conv_state, q_start, n_new,      \
                                                               slot_ids, C, K);                                        \
      rc = llmrs_launch_status("gated_delta (convolution state)");                                                     \
      if (rc != 0) return rc;                                                                                          \
    }                                                                                                                  \
    if (chunked) {                                                                                                     \
      rc = launch_chunked(pq, pk, pv, pbeta, plg, tables, state, q_start, n_new, slot_ids, o_raw, n_requests,          \
                          max_chunks, G, H, d, dv, stream);                                                            \
      if (rc != 0) return rc;                                                                                          \
    } else if (dmax == 32) LLMRS_GD_REC(32, (LLMRS_GD_LANES < 8 ? LLMRS_GD_LANES : 8));                                \
    else if (dmax == 64) LLMRS_GD_REC(64, LLMRS_GD_LANES);                                                             \
    else if (dmax == 128) LLMRS_GD_REC(128, LLMRS_GD_LANES);                                                           \
    else LLMRS_GD_REC(256, LLMRS_GD_LANES);                                                                            \
    rc = llmrs_launch_status("gated_delta (recurrence)");                                                              \
    if (rc != 0) return rc;                                                                                            \
    gdr_out_kernel<T><<<(rows + 3) / 4, 128, 0, stream>>>(o_raw, (const T*)gate, gate_stride, norm_w, (T*)out,         \
                                                          out_stride, rows, H, dv, norm_eps, out_scale);               \
  } while (0)
  if (dtype == LLMRS_F32) LLMRS_GD_LAUNCH(float);
  else if (dtype == LLMRS_BF16) LLMRS_GD_LAUNCH(__nv_bfloat16);
  else return llmrs_fail("gated_delta: unknown dtype %d", dtype);
#undef LLMRS_GD_LAUNCH
#undef LLMRS_GD_REC
  return llmrs_launch_status("gated_delta (norm and gate)");
}
