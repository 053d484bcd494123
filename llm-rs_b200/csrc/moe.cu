// Routing and grouping for mixtures of experts.
//
// A router fills, per assignment a = token * top + k, the expert it names and its weight. The sort kernel then
// orders the assignments by expert (a counting sort that keeps token order inside an expert), cuts every expert's
// run into tiles of rows for the grouped matrix product (gemm_grouped.cu) and tells each assignment where its row
// went; the combine kernel sums a token's rows in the order of k with their weights, in float32. Everything stays on
// the device, so steps replay from CUDA graphs.
#include "common.cuh"

// ---------------------------------------------------------------------------------
// Router "table": token id -> a row of `top` expert ids, every expert weighted 1 / top.
// ---------------------------------------------------------------------------------
__global__ void moe_route_table_kernel(const int* __restrict__ token_ids, const int* __restrict__ table,
                                       int* __restrict__ expert_of, float* __restrict__ weight_of, int n_assign,
                                       int top, int vocab, int n_experts) {
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= n_assign) return;
  int id = token_ids[a / top];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  int e = table[(size_t)id * top + a % top];
  e = e < 0 ? 0 : (e >= n_experts ? n_experts - 1 : e);
  expert_of[a] = e;
  weight_of[a] = 1.0f / (float)top;
}

LLMRS_API int llmrs_moe_route_table(const int* token_ids, const int* table, int* expert_of, float* weight_of,
                                    int n_tokens, int top, int vocab, int n_experts, cudaStream_t stream) {
  LLMRS_REQUIRE(n_tokens >= 0 && top > 0 && vocab > 0 && n_experts > 0, "moe_route_table: bad sizes");
  const int n = n_tokens * top;
  if (n == 0) return 0;
  moe_route_table_kernel<<<(n + 255) / 256, 256, 0, stream>>>(token_ids, table, expert_of, weight_of, n, top, vocab,
                                                             n_experts);
  return llmrs_launch_status("moe_route_table");
}

// ---------------------------------------------------------------------------------
// Counting sort of the assignments by expert, one block. Warp w owns a contiguous run of assignments; inside a
// warp's batch of 32 the lanes that name the same expert find their order with match_any. counts[w][e] first holds
// what warp w has seen of expert e, then (after the scan over w) where warp w's rows of expert e begin.
//   row_of[a]     sorted row of assignment a
//   src_token[r]  token whose activations sorted row r reads
//   tiles[i]      (expert, first row, rows) for the grouped product, rows <= tile_rows; *n_tiles of them
// ---------------------------------------------------------------------------------
constexpr int MOE_SORT_THREADS = 1024, MOE_SORT_WARPS = MOE_SORT_THREADS / 32;

__global__ void __launch_bounds__(MOE_SORT_THREADS)
moe_sort_kernel(const int* __restrict__ expert_of, int* __restrict__ row_of, int* __restrict__ src_token,
                int* __restrict__ tiles, int* __restrict__ n_tiles, int n_assign, int top, int n_experts,
                int tile_rows, int tiled) {
  extern __shared__ int sm[];
  int* counts = sm;                                   // [warps][experts]
  int* start = sm + MOE_SORT_WARPS * n_experts;       // [experts + 1]
  int* tile_at = start + n_experts + 1;               // [experts + 1]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < MOE_SORT_WARPS * n_experts; i += MOE_SORT_THREADS) counts[i] = 0;
  __syncthreads();
  const int per_warp = ((n_assign + MOE_SORT_WARPS - 1) / MOE_SORT_WARPS + 31) / 32 * 32;
  const int lo = warp * per_warp, hi = min(n_assign, lo + per_warp);
  int* mine = counts + warp * n_experts;
  for (int base = lo; base < hi; base += 32) {
    const int a = base + lane;
    const bool live = a < hi;
    const int e = live ? expert_of[a] : -1 - lane;    // idle lanes match nobody
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int before = __popc(peers & ((1u << lane) - 1u));
    int seen = 0;
    if (live) seen = mine[e];
    __syncwarp();
    if (live) {
      row_of[a] = seen + before;                      // order inside (warp, expert); completed below
      if (before == 0) mine[e] = seen + __popc(peers);
    }
    __syncwarp();
  }
  __syncthreads();
  for (int e = tid; e < n_experts; e += MOE_SORT_THREADS) {
    int total = 0;
    for (int w = 0; w < MOE_SORT_WARPS; ++w) {
      const int c = counts[w * n_experts + e];
      counts[w * n_experts + e] = total;
      total += c;
    }
    start[e + 1] = total;                             // for now: the expert's number of rows
  }
  __syncthreads();
  if (tid == 0) {
    int rows = 0, t = 0;
    start[0] = 0;
    for (int e = 0; e < n_experts; ++e) {
      const int c = start[e + 1];
      tile_at[e] = t;
      if (e < tiled) t += (c + tile_rows - 1) / tile_rows;      // groups from `tiled` on run no product: no tiles
      rows += c;
      start[e + 1] = rows;
    }
    tile_at[n_experts] = t;
    *n_tiles = t;
  }
  __syncthreads();
  for (int e = tid; e < tiled; e += MOE_SORT_THREADS) {
    const int first = start[e], c = start[e + 1] - first;
    for (int i = 0, t = tile_at[e]; i < c; i += tile_rows, ++t) {
      tiles[3 * t] = e;
      tiles[3 * t + 1] = first + i;
      tiles[3 * t + 2] = min(tile_rows, c - i);
    }
  }
  for (int a = lo + lane; a < hi; a += 32) {
    const int e = expert_of[a];
    const int row = start[e] + mine[e] + row_of[a];
    row_of[a] = row;
    src_token[row] = a / top;
  }
}

// `tiled_groups`: only the first so many groups get tiles (the others' rows are sorted but run no product; an identity
// expert); negative: all.
LLMRS_API int llmrs_moe_sort(const int* expert_of, int* row_of, int* src_token, int* tiles, int* n_tiles,
                             int n_assign, int top, int n_experts, int tile_rows, int tiled_groups,
                             cudaStream_t stream) {
  const int tiled = tiled_groups < 0 || tiled_groups > n_experts ? n_experts : tiled_groups;
  LLMRS_REQUIRE(n_assign >= 0 && top > 0 && tile_rows > 0, "moe_sort: bad sizes");
  LLMRS_REQUIRE(n_experts > 0 && n_experts <= 256, "moe_sort: 1 to 256 experts, got %d", n_experts);
  if (n_assign == 0) return 0;
  const size_t smem = ((size_t)MOE_SORT_WARPS * n_experts + 2 * (n_experts + 1)) * sizeof(int);
  moe_sort_kernel<<<1, MOE_SORT_THREADS, smem, stream>>>(expert_of, row_of, src_token, tiles, n_tiles, n_assign, top,
                                                         n_experts, tile_rows, tiled);
  return llmrs_launch_status("moe_sort");
}

// ---------------------------------------------------------------------------------
// out[t, :] = sum_k weight_of[t * top + k] * rows[row_of[t * top + k], :], k in order, float32.
// ---------------------------------------------------------------------------------
template <typename TO>
__global__ void moe_combine_kernel(const float* __restrict__ rows, const int* __restrict__ row_of,
                                   const float* __restrict__ weight_of, TO* __restrict__ out, int top, int width) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float s = 0.f;
    for (int k = 0; k < top; ++k)
      s = fmaf(weight_of[t * top + k], rows[(size_t)row_of[t * top + k] * width + c], s);
    out[(size_t)t * width + c] = from_float<TO>(s);
  }
}

LLMRS_API int llmrs_moe_combine(const float* rows, const int* row_of, const float* weight_of, void* out,
                                int out_dtype, int n_tokens, int top, int width, cudaStream_t stream) {
  LLMRS_REQUIRE(n_tokens >= 0 && top > 0 && width > 0, "moe_combine: bad sizes");
  if (n_tokens == 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
  if (out_dtype == LLMRS_F32)
    moe_combine_kernel<float><<<n_tokens, threads, 0, stream>>>(rows, row_of, weight_of, (float*)out, top, width);
  else if (out_dtype == LLMRS_BF16)
    moe_combine_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(rows, row_of, weight_of,
                                                                        (__nv_bfloat16*)out, top, width);
  else
    return llmrs_fail("moe_combine: unknown dtype %d", out_dtype);
  return llmrs_launch_status("moe_combine");
}

// ---------------------------------------------------------------------------------
// Router "linear": the `top` largest of a token's logits (float32, made by a product before this kernel), weighted
// by the softmax over the chosen logits only. One warp per token; the lanes hold the logits strided and pick the
// largest `top` times (among equal logits the lower expert wins), so the assignments come in order of falling logit.
// ---------------------------------------------------------------------------------
constexpr int ROUTE_PER_LANE = 8;      // up to 256 experts

__global__ void moe_route_top_kernel(const float* __restrict__ logits, long long stride, int* __restrict__ expert_of,
                                     float* __restrict__ weight_of, int n_tokens, int n_experts, int top) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= n_tokens) return;
  float z[ROUTE_PER_LANE];
#pragma unroll
  for (int j = 0; j < ROUTE_PER_LANE; ++j) {
    const int e = lane + 32 * j;
    z[j] = e < n_experts ? logits[(size_t)t * stride + e] : -INFINITY;
  }
  float first = 0.f, sum = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < ROUTE_PER_LANE; ++j) {
      const int e = lane + 32 * j;
      if (e < n_experts && (z[j] > best || (z[j] == best && e < at)) && z[j] != -INFINITY) { best = z[j]; at = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at == 0x7fffffff) at = k;      // logits that are no numbers: any expert, weight 0
#pragma unroll
    for (int j = 0; j < ROUTE_PER_LANE; ++j)
      if (lane + 32 * j == at) z[j] = -INFINITY;
    if (k == 0) first = best;
    const float p = expf(best - first);       // the first pick is the largest: no overflow
    sum += p;
    if (lane == 0) {
      expert_of[(size_t)t * top + k] = at;
      weight_of[(size_t)t * top + k] = p;
    }
  }
  __syncwarp();
  if (lane < top) weight_of[(size_t)t * top + lane] /= sum;
  for (int k = 32 + lane; k < top; k += 32) weight_of[(size_t)t * top + k] /= sum;
}

LLMRS_API int llmrs_moe_route_top(const float* logits, long long stride, int* expert_of, float* weight_of,
                                  int n_tokens, int n_experts, int top, cudaStream_t stream) {
  LLMRS_REQUIRE(n_tokens >= 0 && top > 0 && top <= n_experts, "moe_route_top: bad sizes");
  LLMRS_REQUIRE(n_experts <= 32 * ROUTE_PER_LANE, "moe_route_top: at most %d experts, got %d", 32 * ROUTE_PER_LANE,
                n_experts);
  if (n_tokens == 0) return 0;
  moe_route_top_kernel<<<(n_tokens + 3) / 4, 128, 0, stream>>>(logits, stride, expert_of, weight_of, n_tokens,
                                                              n_experts, top);
  return llmrs_launch_status("moe_route_top");
}

// ---------------------------------------------------------------------------------
// moe_combine plus an expert that every token uses:
// out[t, :] = sum_k weight_of[t, k] * rows[row_of[t, k], :] + sigmoid(gate[t]) * shared[t, :]   (gate null: factor 1)
// ---------------------------------------------------------------------------------
template <typename TS>
__global__ void moe_combine_shared_kernel(const float* __restrict__ rows, const int* __restrict__ row_of,
                                          const float* __restrict__ weight_of, const TS* __restrict__ shared,
                                          const float* __restrict__ gate, long long gate_stride,
                                          float* __restrict__ out, int top, int width) {
  const int t = blockIdx.x;
  const float g = shared == nullptr ? 0.f : (gate ? 1.0f / (1.0f + expf(-gate[(size_t)t * gate_stride])) : 1.0f);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float s = 0.f;
    for (int k = 0; k < top; ++k)
      s = fmaf(weight_of[t * top + k], rows[(size_t)row_of[t * top + k] * width + c], s);
    if (shared) s = fmaf(g, to_float(shared[(size_t)t * width + c]), s);
    out[(size_t)t * width + c] = s;
  }
}

LLMRS_API int llmrs_moe_combine_shared(const float* rows, const int* row_of, const float* weight_of,
                                       const void* shared, int shared_dtype, const float* gate, long long gate_stride,
                                       float* out, int n_tokens, int top, int width, cudaStream_t stream) {
  LLMRS_REQUIRE(n_tokens >= 0 && top > 0 && width > 0, "moe_combine_shared: bad sizes");
  if (n_tokens == 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
  if (shared == nullptr || shared_dtype == LLMRS_F32)
    moe_combine_shared_kernel<float><<<n_tokens, threads, 0, stream>>>(rows, row_of, weight_of, (const float*)shared,
                                                                       gate, gate_stride, out, top, width);
  else if (shared_dtype == LLMRS_BF16)
    moe_combine_shared_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
        rows, row_of, weight_of, (const __nv_bfloat16*)shared, gate, gate_stride, out, top, width);
  else
    return llmrs_fail("moe_combine_shared: unknown dtype %d", shared_dtype);
  return llmrs_launch_status("moe_combine_shared");
}

// ---------------------------------------------------------------------------------
// Router "softmax_bias": scores s = softmax(logits) over ALL experts; the `top` experts with the largest s + bias are
// chosen (among equals the lower expert), and their weights are the scores s themselves, not renormalised. The last
// experts (from `n_real` on) are identity experts: they have no weights of their own and are all reported as group
// `n_real`, whose rows run no product. One warp per token, assignments in order of falling choice score.
// ---------------------------------------------------------------------------------
__global__ void moe_route_biased_kernel(const float* __restrict__ logits, long long stride,
                                        const float* __restrict__ bias, int* __restrict__ expert_of,
                                        float* __restrict__ weight_of, int n_tokens, int n_all, int n_real, int top) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= n_tokens) return;
  float s[ROUTE_PER_LANE], c[ROUTE_PER_LANE];
  float m = -INFINITY;
#pragma unroll
  for (int j = 0; j < ROUTE_PER_LANE; ++j) {
    const int e = lane + 32 * j;
    s[j] = e < n_all ? logits[(size_t)t * stride + e] : -INFINITY;
    m = fmaxf(m, s[j]);
  }
  m = warp_max(m);
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < ROUTE_PER_LANE; ++j) {
    s[j] = lane + 32 * j < n_all ? expf(s[j] - m) : 0.f;
    sum += s[j];
  }
  sum = warp_sum(sum);
#pragma unroll
  for (int j = 0; j < ROUTE_PER_LANE; ++j) {
    const int e = lane + 32 * j;
    s[j] = s[j] / sum;
    c[j] = e < n_all ? s[j] + (bias ? bias[e] : 0.f) : -INFINITY;
  }
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY, score = 0.f;
    int at = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < ROUTE_PER_LANE; ++j) {
      const int e = lane + 32 * j;
      if (e < n_all && c[j] != -INFINITY && (c[j] > best || (c[j] == best && e < at))) { best = c[j]; at = e; score = s[j]; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      const float os = __shfl_xor_sync(0xffffffffu, score, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; score = os; }
    }
    if (at == 0x7fffffff) { at = k; score = 0.f; }      // logits that are no numbers: any expert, weight 0
#pragma unroll
    for (int j = 0; j < ROUTE_PER_LANE; ++j)
      if (lane + 32 * j == at) c[j] = -INFINITY;
    if (lane == 0) {
      expert_of[(size_t)t * top + k] = at < n_real ? at : n_real;
      weight_of[(size_t)t * top + k] = score;
    }
  }
}

LLMRS_API int llmrs_moe_route_biased(const float* logits, long long stride, const float* bias, int* expert_of,
                                     float* weight_of, int n_tokens, int n_all, int n_real, int top,
                                     cudaStream_t stream) {
  LLMRS_REQUIRE(n_tokens >= 0 && top > 0 && top <= n_all && n_real >= 0 && n_real <= n_all,
                "moe_route_biased: bad sizes");
  LLMRS_REQUIRE(n_all <= 32 * ROUTE_PER_LANE, "moe_route_biased: at most %d experts, got %d", 32 * ROUTE_PER_LANE,
                n_all);
  if (n_tokens == 0) return 0;
  moe_route_biased_kernel<<<(n_tokens + 3) / 4, 128, 0, stream>>>(logits, stride, bias, expert_of, weight_of,
                                                                 n_tokens, n_all, n_real, top);
  return llmrs_launch_status("moe_route_biased");
}

// ---------------------------------------------------------------------------------
// moe_combine where an assignment to group `n_real` (an identity expert) stands for the token's own input row:
// out[t, :] = sum_k weight_of[t, k] * (expert_of[t, k] < n_real ? rows[row_of[t, k], :] : x[t, :]), k in order.
// ---------------------------------------------------------------------------------
template <typename TX>
__global__ void moe_combine_identity_kernel(const float* __restrict__ rows, const int* __restrict__ row_of,
                                            const float* __restrict__ weight_of, const int* __restrict__ expert_of,
                                            const TX* __restrict__ x, float* __restrict__ out, int top, int width,
                                            int n_real) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float s = 0.f;
    for (int k = 0; k < top; ++k) {
      const int a = t * top + k;
      const float v = expert_of[a] < n_real ? rows[(size_t)row_of[a] * width + c] : to_float(x[(size_t)t * width + c]);
      s = fmaf(weight_of[a], v, s);
    }
    out[(size_t)t * width + c] = s;
  }
}

LLMRS_API int llmrs_moe_combine_identity(const float* rows, const int* row_of, const float* weight_of,
                                         const int* expert_of, const void* x, int x_dtype, float* out, int n_tokens,
                                         int top, int width, int n_real, cudaStream_t stream) {
  LLMRS_REQUIRE(n_tokens >= 0 && top > 0 && width > 0, "moe_combine_identity: bad sizes");
  if (n_tokens == 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
  if (x_dtype == LLMRS_F32)
    moe_combine_identity_kernel<float><<<n_tokens, threads, 0, stream>>>(rows, row_of, weight_of, expert_of,
                                                                         (const float*)x, out, top, width, n_real);
  else if (x_dtype == LLMRS_BF16)
    moe_combine_identity_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
        rows, row_of, weight_of, expert_of, (const __nv_bfloat16*)x, out, top, width, n_real);
  else
    return llmrs_fail("moe_combine_identity: unknown dtype %d", x_dtype);
  return llmrs_launch_status("moe_combine_identity");
}
