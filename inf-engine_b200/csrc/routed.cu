// A mixture of feed-forward experts on the device, without a trip to the host:
//   route    per token, from float32 router logits: sigmoid scores, a correction added for the choice only, the best
//            groups of neighbouring experts kept, the top experts among them, their normalised weights, and the
//            shared expert's gate;
//   sort     the (token, choice) pairs ordered by expert, and a table of row tiles, none of which spans two experts;
//   product  C[pair] = A[token of pair] W[expert of pair]^T over those tiles on CUDA cores (float32 products and
//            sums, every output one accumulator that walks k upward, so a row's result does not depend on which
//            tile or step it is in), optionally with silu(gate) * up in the epilogue;
//   combine  out[token] = sum over its choices of weight * y[pair] + gate * shared[token], choices in order.
#include "common.cuh"

// ------------------------------------------------------------------ route
// One warp per token.  logits [n, ld]: columns 0..E-1 the experts, column `gate_col` (if >= 0) the shared expert's
// gate.  Ties go to the lower index.
template <typename TW>
__global__ void __launch_bounds__(128)
route_kernel(const float* __restrict__ logits, int ld, const TW* __restrict__ correction, int* __restrict__ ids,
             float* __restrict__ weights, float* __restrict__ gate, int n_tokens, int n_experts, int top, int n_groups,
             int keep_groups, float route_scale, float weight_eps, int gate_col) {
  extern __shared__ float sm[];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= n_tokens) return;
  float* score = sm + (size_t)warp * (2 * n_experts + n_groups);   // s
  float* choice = score + n_experts;                               // s + correction, -inf once taken or shut out
  float* gscore = choice + n_experts;
  const float* z = logits + (size_t)t * ld;
  for (int e = lane; e < n_experts; e += 32) {
    const float s = 1.f / (1.f + expf(-z[e]));
    score[e] = s;
    choice[e] = s + (correction ? to_f32(correction[e]) : 0.f);
  }
  __syncwarp();
  const int per = n_experts / n_groups;
  if (keep_groups < n_groups) {
    for (int g = lane; g < n_groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;          // the two largest of the group
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float c = choice[e];
        if (c > a) { b = a; a = c; } else if (c > b) b = c;
      }
      gscore[g] = per > 1 ? a + b : a;
    }
    __syncwarp();
    // the groups that stay: keep_groups times the largest score left; the others are shut out afterwards
    for (int r = 0; r < keep_groups; ++r) {
      float best = -INFINITY;
      int at = 0x7fffffff;
      for (int g = lane; g < n_groups; g += 32) {
        const float c = gscore[g];
        if (c != INFINITY && (c > best || (c == best && g < at))) { best = c; at = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
      }
      if (lane == 0 && at != 0x7fffffff) gscore[at] = INFINITY;      // marks a kept group
      __syncwarp();
    }
    for (int e = lane; e < n_experts; e += 32)
      if (gscore[e / per] != INFINITY) choice[e] = -INFINITY;
    __syncwarp();
  }
  float total = 0.f;
  for (int r = 0; r < top; ++r) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < n_experts; e += 32) {
      const float c = choice[e];
      if (c > best || (c == best && e < at && c != -INFINITY)) { best = c; at = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at == 0x7fffffff) at = 0;             // nothing left to choose (scores that are not numbers): expert 0, weight as it is
    const float s = score[at];
    total += s;
    if (lane == 0) {
      ids[(size_t)t * top + r] = at;
      weights[(size_t)t * top + r] = s;
      choice[at] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane == 0) {
    const float f = route_scale / (total + weight_eps);
    for (int r = 0; r < top; ++r) weights[(size_t)t * top + r] *= f;
    if (gate != nullptr) gate[t] = gate_col >= 0 ? 1.f / (1.f + expf(-z[gate_col])) : 1.f;
  }
}

extern "C" int ie_moe_route(const float* logits, int ld, const void* correction, int w_dtype, int* ids, float* weights,
                            float* gate, int n_tokens, int n_experts, int top, int n_groups, int keep_groups,
                            float route_scale, float weight_eps, int gate_col, cudaStream_t stream) {
  if (n_tokens <= 0) return IE_OK;
  if (n_experts <= 0 || top <= 0 || top > n_experts || n_groups <= 0 || n_experts % n_groups || keep_groups <= 0 ||
      keep_groups > n_groups)
    return IE_BAD_SIZE;
  const size_t smem = sizeof(float) * 4 * (size_t)(2 * n_experts + n_groups);
  if (smem > 47 * 1024) return IE_BAD_SIZE;
  const unsigned blocks = (unsigned)((n_tokens + 3) / 4);
  if (w_dtype == IE_F32)
    return launch_k(route_kernel<float>, blocks, 128, smem, stream, logits, ld, (const float*)correction, ids, weights,
                    gate, n_tokens, n_experts, top, n_groups, keep_groups, route_scale, weight_eps, gate_col);
  if (w_dtype == IE_BF16)
    return launch_k(route_kernel<bf16>, blocks, 128, smem, stream, logits, ld, (const bf16*)correction, ids, weights,
                    gate, n_tokens, n_experts, top, n_groups, keep_groups, route_scale, weight_eps, gate_col);
  return IE_BAD_DTYPE;
}

// ------------------------------------------------------------------ sort
// One block.  sorted[pos] = pair index (token * top + choice) with the pairs of expert 0 first, then expert 1, ...;
// tiles[4 * i .. 4 * i + 3] = (expert, first position, rows, 0) for every tile of at most `tile_rows` rows; tiles
// beyond the last carry rows = 0.  The order of an expert's pairs among themselves is whatever the atomics give:
// a pair's result does not depend on its place.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ ids, int n_pairs, int n_experts, int tile_rows, int* __restrict__ sorted,
                int* __restrict__ tiles, int max_tiles) {
  extern __shared__ int si[];
  int* count = si;
  int* offset = si + n_experts;
  int* cursor = si + 2 * n_experts;
  pdl_trigger();
  pdl_wait();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) count[e] = cursor[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < n_experts) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int pos = 0, nt = 0;
    for (int e = 0; e < n_experts; ++e) {
      offset[e] = pos;
      for (int r = 0; r < count[e] && nt < max_tiles; r += tile_rows, ++nt) {
        tiles[4 * nt] = e;
        tiles[4 * nt + 1] = pos + r;
        tiles[4 * nt + 2] = min(tile_rows, count[e] - r);
        tiles[4 * nt + 3] = 0;
      }
      pos += count[e];
    }
    for (; nt < max_tiles; ++nt) tiles[4 * nt] = tiles[4 * nt + 1] = tiles[4 * nt + 2] = tiles[4 * nt + 3] = 0;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < n_experts) sorted[offset[e] + atomicAdd(&cursor[e], 1)] = p;
  }
}

extern "C" int ie_moe_sort(const int* ids, int n_pairs, int n_experts, int tile_rows, int* sorted, int* tiles,
                           int max_tiles, cudaStream_t stream) {
  if (n_pairs <= 0) return IE_OK;
  if (n_experts <= 0 || tile_rows <= 0 || 3 * (size_t)n_experts * sizeof(int) > 47 * 1024) return IE_BAD_SIZE;
  return launch_k(moe_sort_kernel, 1, 1024, 3 * (size_t)n_experts * sizeof(int), stream, ids, n_pairs, n_experts,
                  tile_rows, sorted, tiles, max_tiles);
}

// ------------------------------------------------------------------ grouped product
#define MG_BM 64
#define MG_BN 64
#define MG_BK 16
#define MG_THREADS 256

// A row of tile (expert e, positions pos0 .. pos0 + rows): gather = 1: row sorted[pos] / top of A (a token's
// activations); gather = 0: row pos of A (what the product before left in sorted order).  C row: scatter = 1: row
// sorted[pos] (the pair's own place), else row pos.  W is [experts, N, K].  epi 1: columns alternate gate, up and the
// output is silu(gate) * up, N / 2 wide.
template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(MG_THREADS)
moe_gemm_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TC* __restrict__ C, const int* __restrict__ sorted,
                const int* __restrict__ tiles, int N, int K, int lda, int ldc, long long w_expert_stride, int top,
                int gather, int scatter, int epi) {
  pdl_trigger();
  pdl_wait();
  __shared__ float As[MG_BK][MG_BM + 4];
  __shared__ float Ws[MG_BK][MG_BN + 4];
  __shared__ int a_row[MG_BM], c_row[MG_BM];
  const int tile = blockIdx.y;
  const int rows = tiles[4 * tile + 2];
  if (rows <= 0) return;
  const int expert = tiles[4 * tile], pos0 = tiles[4 * tile + 1];
  const int n0 = blockIdx.x * MG_BN;
  const int tid = threadIdx.x;
  if (tid < MG_BM) {
    int ar = -1, cr = -1;
    if (tid < rows) {
      const int pair = sorted[pos0 + tid];
      ar = gather ? pair / top : pos0 + tid;
      cr = scatter ? pair : pos0 + tid;
    }
    a_row[tid] = ar;
    c_row[tid] = cr;
  }
  __syncthreads();
  const TW* Wexp = W + (size_t)expert * w_expert_stride;
  const int tx = tid & 15, ty = tid >> 4;
  const int lr = tid >> 2, lc = (tid & 3) * 4;
  const int my_a = a_row[lr];
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += MG_BK) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = k0 + lc + u;
      const int wn = n0 + lr;
      As[lc + u][lr] = (my_a >= 0 && k < K) ? to_f32(A[(size_t)my_a * lda + k]) : 0.f;
      Ws[lc + u][lr] = (wn < N && k < K) ? to_f32(Wexp[(size_t)wn * K + k]) : 0.f;
    }
    __syncthreads();
#ifdef IE_SIMT_CHAIN
#pragma unroll
    for (int kk = 0; kk < MG_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
#else
    // the slab's 16 products are summed by themselves and then added to the total: the rounding of a long sum
    // grows with K / 16 + 16 steps instead of K
    float part[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) part[i][j] = 0.f;
#pragma unroll
    for (int kk = 0; kk < MG_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) part[i][j] = fmaf(a[i], b[j], part[i][j]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] += part[i][j];
#endif
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int cr = c_row[ty * 4 + i];
    if (cr < 0) continue;
    if (epi == 1) {
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        const int n = n0 + tx * 4 + j;
        if (n + 1 < N) {
          const float g = acc[i][j];
          C[(size_t)cr * ldc + (n >> 1)] = from_f32<TC>(g / (1.f + expf(-g)) * acc[i][j + 1]);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + tx * 4 + j;
        if (n < N) C[(size_t)cr * ldc + n] = from_f32<TC>(acc[i][j]);
      }
    }
  }
}

template <typename TA, typename TW, typename TC>
static int launch_moe_gemm(const void* A, const void* W, void* C, const int* sorted, const int* tiles, int max_tiles,
                           int N, int K, int lda, int ldc, long long wes, int top, int gather, int scatter, int epi,
                           cudaStream_t stream) {
  dim3 grid((N + MG_BN - 1) / MG_BN, max_tiles);
  return launch_k(moe_gemm_kernel<TA, TW, TC>, grid, MG_THREADS, 0, stream, (const TA*)A, (const TW*)W, (TC*)C, sorted,
                  tiles, N, K, lda, ldc, wes, top, gather, scatter, epi);
}

extern "C" int ie_moe_tile_rows() { return MG_BM; }

extern "C" int ie_moe_gemm(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype,
                           const int* sorted, const int* tiles, int max_tiles, int N, int K, int lda, int ldc,
                           long long w_expert_stride, int top, int gather, int scatter, int epi, cudaStream_t stream) {
  if (max_tiles <= 0 || N <= 0) return IE_OK;
  if (K <= 0 || top <= 0 || (epi == 1 && (N & 1))) return IE_BAD_SIZE;
  const int code = a_dtype * 4 + w_dtype * 2 + c_dtype;
#define MG_GO(TA, TW, TC)                                                                                         \
  return launch_moe_gemm<TA, TW, TC>(A, W, C, sorted, tiles, max_tiles, N, K, lda, ldc, w_expert_stride, top, gather, \
                                     scatter, epi, stream)
  switch (code) {
    case 0: MG_GO(float, float, float);
    case 2: MG_GO(float, bf16, float);
    case 4: MG_GO(bf16, float, float);
    case 5: MG_GO(bf16, float, bf16);
    case 6: MG_GO(bf16, bf16, float);
    case 7: MG_GO(bf16, bf16, bf16);
    default: return IE_BAD_DTYPE;
  }
#undef MG_GO
}

// ------------------------------------------------------------------ combine
// out[t, :] = sum_r weights[t, r] * y[t * top + r, :]  (r upward)  + gate[t] * shared[t, :]
template <typename TS>
__global__ void moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ weights,
                                   const float* __restrict__ gate, const TS* __restrict__ shared_out, int shared_stride,
                                   float* __restrict__ out, int d, int top) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const float* w = weights + (size_t)t * top;
  const float g = (gate != nullptr && shared_out != nullptr) ? gate[t] : 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < top; ++r) acc = fmaf(w[r], y[((size_t)t * top + r) * d + i], acc);
    if (shared_out != nullptr) acc = fmaf(g, to_f32(shared_out[(size_t)t * shared_stride + i]), acc);
    out[(size_t)t * d + i] = acc;
  }
}

extern "C" int ie_moe_combine(const float* y, const float* weights, const float* gate, const void* shared_out,
                              int shared_dtype, int shared_stride, float* out, int n_tokens, int d, int top,
                              cudaStream_t stream) {
  if (n_tokens <= 0) return IE_OK;
  const int threads = d >= 1024 ? 256 : 128;
  if (shared_out == nullptr || shared_dtype == IE_F32)
    return launch_k(moe_combine_kernel<float>, n_tokens, threads, 0, stream, y, weights, gate,
                    (const float*)shared_out, shared_stride, out, d, top);
  if (shared_dtype == IE_BF16)
    return launch_k(moe_combine_kernel<bf16>, n_tokens, threads, 0, stream, y, weights, gate, (const bf16*)shared_out,
                    shared_stride, out, d, top);
  return IE_BAD_DTYPE;
}
