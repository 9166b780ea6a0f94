// Row-wise kernels for parts beyond the plain Llama block: LayerNorm with weight and bias fused with the
// residual sum, a hashed bigram embedding added to the token embedding, a bias added to a product, the
// PolyNorm activation, and a per-head RMS norm of queries and keys fused with the write of keys and values
// into cache pages.  Statistics and sums are float32 whatever the activation type is.
#include "common.cuh"

// ------------------------------------------------------------------ LayerNorm
// x = residual[row] (+ delta[row]);  residual[row] = x (unless rows are gathered);
// out[m] = (x - mean(x)) / sqrt(mean((x - mean)^2) + eps) * weight + bias
// One block per output row; x is staged in shared memory between the passes (mean first, then the squared
// deviations from it, so that a large mean does not cancel the variance).
template <typename TA, typename TW>
__global__ void layernorm_kernel(float* __restrict__ residual, const TA* __restrict__ delta,
                                 const TW* __restrict__ weight, const TW* __restrict__ bias, TA* __restrict__ out,
                                 const int* __restrict__ row_index, int d, float eps) {
  extern __shared__ float xs[];
  __shared__ float red[33];
  pdl_trigger();
  pdl_wait();
  const int m = blockIdx.x;
  const int row = row_index ? row_index[m] : m;
  float* res = residual + (size_t)row * d;
  const TA* del = delta ? delta + (size_t)row * d : nullptr;
  float s = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float x = res[i];
    if (del) x += to_f32(del[i]);
    xs[i] = x;
    s += x;
    if (del && !row_index) res[i] = x;
  }
  const float mean = block_sum(s, red) / (float)d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float c = xs[i] - mean;
    ss += c * c;
  }
  const float sd = sqrtf(block_sum(ss, red) / (float)d + eps);
  TA* o = out + (size_t)m * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float y = (xs[i] - mean) / sd * to_f32(weight[i]) + (bias ? to_f32(bias[i]) : 0.f);
    o[i] = from_f32<TA>(y);
  }
}

template <typename TA, typename TW>
static int launch_layernorm(float* residual, const void* delta, const void* weight, const void* bias, void* out,
                            const int* row_index, int n_rows, int d, float eps, cudaStream_t stream) {
  const size_t smem = (size_t)d * sizeof(float);
  if (smem > 200 * 1024) return IE_BAD_SIZE;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(layernorm_kernel<TA, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
  return launch_k(layernorm_kernel<TA, TW>, n_rows, threads, smem, stream, residual, (const TA*)delta,
                  (const TW*)weight, (const TW*)bias, (TA*)out, row_index, d, eps);
}

extern "C" int ie_layernorm(float* residual, const void* delta, const void* weight, const void* bias, int w_dtype,
                            void* out, int act_dtype, const int* row_index, int n_rows, int d, float eps,
                            cudaStream_t stream) {
  if (n_rows <= 0) return IE_OK;
  if (act_dtype == IE_F32 && w_dtype == IE_F32)
    return launch_layernorm<float, float>(residual, delta, weight, bias, out, row_index, n_rows, d, eps, stream);
  if (act_dtype == IE_F32 && w_dtype == IE_BF16)
    return launch_layernorm<float, bf16>(residual, delta, weight, bias, out, row_index, n_rows, d, eps, stream);
  if (act_dtype == IE_BF16 && w_dtype == IE_F32)
    return launch_layernorm<bf16, float>(residual, delta, weight, bias, out, row_index, n_rows, d, eps, stream);
  if (act_dtype == IE_BF16 && w_dtype == IE_BF16)
    return launch_layernorm<bf16, bf16>(residual, delta, weight, bias, out, row_index, n_rows, d, eps, stream);
  return IE_BAD_DTYPE;
}

// ------------------------------------------------- token embedding + hashed bigram embedding
// residual[n] = table[id[n]] + bigram[row(n)],  row = (prev * mul_prev + id * mul_cur) mod buckets, and row
// `buckets` (the table's last) for the first token of a sequence (position 0).  The previous token of a
// request's first token in this step is what the request's state slot holds (written by the step before); the
// block that reads a slot is the one that then stores the request's last token of this step there, so no
// other block touches the slot.  A negative slot (a padding row) has no state.
template <typename TW>
__global__ void embed_bigram_kernel(const int* __restrict__ ids, const int* __restrict__ positions,
                                    const int* __restrict__ q_start, const int* __restrict__ slots, int n_requests,
                                    const TW* __restrict__ table, const TW* __restrict__ bigram,
                                    int* __restrict__ prev_state, float* __restrict__ residual, int d, int vocab,
                                    int buckets, long long mul_prev, long long mul_cur) {
  __shared__ int s_row, s_id;
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  if (threadIdx.x == 0) {
    int lo = 0, hi = n_requests;          // the request r with q_start[r] <= n < q_start[r + 1]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (q_start[mid] <= n) lo = mid; else hi = mid;
    }
    const int r = lo;
    const int first = q_start[r];
    int id = IE_TOKEN(ids[n]);
    if (id < 0 || id >= vocab) id = 0;
    const int slot = slots[r];
    int row = buckets;
    if (positions[n] > 0) {
      int prev = n > first ? ids[n - 1] : (slot >= 0 ? prev_state[slot] : 0);
      if (prev < 0 || prev >= vocab) prev = 0;
      long long hsh = ((long long)prev * mul_prev + (long long)id * mul_cur) % (long long)buckets;
      if (hsh < 0) hsh += buckets;          // the mathematical remainder, also for a negative multiplier
      row = (int)hsh;
    }
    if (n == first && slot >= 0) prev_state[slot] = ids[q_start[r + 1] - 1];
    s_row = row;
    s_id = id;
  }
  __syncthreads();
  const TW* a = table + (size_t)s_id * d;
  const TW* b = bigram + (size_t)s_row * d;
  float* out = residual + (size_t)n * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) out[i] = to_f32(a[i]) + to_f32(b[i]);
}

extern "C" int ie_embed_bigram(const int* ids, const int* positions, const int* q_start, const int* slots,
                               int n_requests, const void* table, const void* bigram, int table_dtype,
                               int* prev_state, float* residual, int n_tokens, int d, int vocab, int buckets,
                               long long mul_prev, long long mul_cur, cudaStream_t stream) {
  if (n_tokens <= 0) return IE_OK;
  if (buckets <= 0 || n_requests <= 0) return IE_BAD_SIZE;
  const int threads = d >= 1024 ? 256 : 128;
  if (table_dtype == IE_F32)
    return launch_k(embed_bigram_kernel<float>, n_tokens, threads, 0, stream, ids, positions, q_start, slots,
                    n_requests, (const float*)table, (const float*)bigram, prev_state, residual, d, vocab, buckets,
                    mul_prev, mul_cur);
  if (table_dtype == IE_BF16)
    return launch_k(embed_bigram_kernel<bf16>, n_tokens, threads, 0, stream, ids, positions, q_start, slots,
                    n_requests, (const bf16*)table, (const bf16*)bigram, prev_state, residual, d, vocab, buckets,
                    mul_prev, mul_cur);
  return IE_BAD_DTYPE;
}

// ------------------------------------------------------------------ bias of a product
// out[n, j] += bias[j]
template <typename TA, typename TW>
__global__ void add_bias_kernel(TA* __restrict__ out, const TW* __restrict__ bias, int cols, int stride, size_t total) {
  pdl_trigger();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t n = idx / cols;
  const int j = (int)(idx - n * cols);
  TA* p = out + n * stride + j;
  *p = from_f32<TA>(to_f32(*p) + to_f32(bias[j]));
}

extern "C" int ie_add_bias(void* out, int out_dtype, const void* bias, int bias_dtype, int n_rows, int cols,
                           int stride, cudaStream_t stream) {
  const size_t total = (size_t)n_rows * cols;
  if (total == 0) return IE_OK;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  const int code = out_dtype * 2 + bias_dtype;
  switch (code) {
    case 0: return launch_k(add_bias_kernel<float, float>, blocks, 256, 0, stream, (float*)out, (const float*)bias, cols, stride, total);
    case 1: return launch_k(add_bias_kernel<float, bf16>, blocks, 256, 0, stream, (float*)out, (const bf16*)bias, cols, stride, total);
    case 2: return launch_k(add_bias_kernel<bf16, float>, blocks, 256, 0, stream, (bf16*)out, (const float*)bias, cols, stride, total);
    case 3: return launch_k(add_bias_kernel<bf16, bf16>, blocks, 256, 0, stream, (bf16*)out, (const bf16*)bias, cols, stride, total);
    default: return IE_BAD_DTYPE;
  }
}

// ------------------------------------------------------------------ tanh
// out[n, j] = tanh(in[n, j]); `in` is row-strided (columns of a wider buffer), `out` contiguous
template <typename TA>
__global__ void tanh_kernel(const TA* __restrict__ in, TA* __restrict__ out, int cols, int in_stride, size_t total) {
  pdl_trigger();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t n = idx / cols;
  const int j = (int)(idx - n * cols);
  out[idx] = from_f32<TA>(tanhf(to_f32(in[n * in_stride + j])));
}

extern "C" int ie_tanh(const void* in, void* out, int n_rows, int cols, int in_stride, int act_dtype,
                       cudaStream_t stream) {
  const size_t total = (size_t)n_rows * cols;
  if (total == 0) return IE_OK;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (act_dtype == IE_F32)
    return launch_k(tanh_kernel<float>, blocks, 256, 0, stream, (const float*)in, (float*)out, cols, in_stride, total);
  if (act_dtype == IE_BF16)
    return launch_k(tanh_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)in, (bf16*)out, cols, in_stride, total);
  return IE_BAD_DTYPE;
}

// ------------------------------------------------------------------ PolyNorm activation
// z = in[n] (+ bias);  N(x) = x / sqrt(mean(x^2) + eps) over the row;
// out[n] = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3, powers element by element; coef = {c0, c1, c2, c3} on the device.
// One block per row; z is staged in shared memory between the sums and the write.
template <typename TA, typename TW>
__global__ void polynorm_kernel(const TA* __restrict__ in, const TW* __restrict__ bias, const TW* __restrict__ coef,
                                TA* __restrict__ out, int cols, int in_stride, float eps) {
  extern __shared__ float zs[];
  __shared__ float red[33];
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  const TA* row = in + (size_t)n * in_stride;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) {
    float z = to_f32(row[i]);
    if (bias) z += to_f32(bias[i]);
    zs[i] = z;
    const float z2 = z * z, z3 = z2 * z;
    s2 += z2;
    s4 += z2 * z2;
    s6 += z3 * z3;
  }
  const float r1 = sqrtf(block_sum(s2, red) / (float)cols + eps);
  const float r2 = sqrtf(block_sum(s4, red) / (float)cols + eps);
  const float r3 = sqrtf(block_sum(s6, red) / (float)cols + eps);
  const float c0 = to_f32(coef[0]), c1 = to_f32(coef[1]), c2 = to_f32(coef[2]), c3 = to_f32(coef[3]);
  TA* o = out + (size_t)n * cols;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) {
    const float z = zs[i];
    const float z2 = z * z;
    o[i] = from_f32<TA>(c0 * (z / r1) + c1 * (z2 / r2) + c2 * (z2 * z / r3) + c3);
  }
}

template <typename TA, typename TW>
static int launch_polynorm(const void* in, const void* bias, const void* coef, void* out, int n_rows, int cols,
                           int in_stride, float eps, cudaStream_t stream) {
  const size_t smem = (size_t)cols * sizeof(float);
  if (smem > 200 * 1024) return IE_BAD_SIZE;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(polynorm_kernel<TA, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int threads = cols >= 4096 ? 512 : (cols >= 512 ? 256 : 128);
  return launch_k(polynorm_kernel<TA, TW>, n_rows, threads, smem, stream, (const TA*)in, (const TW*)bias,
                  (const TW*)coef, (TA*)out, cols, in_stride, eps);
}

extern "C" int ie_polynorm(const void* in, const void* bias, const void* coef, int w_dtype, void* out, int act_dtype,
                           int n_rows, int cols, int in_stride, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return IE_OK;
  if (cols <= 0) return IE_BAD_SIZE;
  if (act_dtype == IE_F32 && w_dtype == IE_F32)
    return launch_polynorm<float, float>(in, bias, coef, out, n_rows, cols, in_stride, eps, stream);
  if (act_dtype == IE_F32 && w_dtype == IE_BF16)
    return launch_polynorm<float, bf16>(in, bias, coef, out, n_rows, cols, in_stride, eps, stream);
  if (act_dtype == IE_BF16 && w_dtype == IE_F32)
    return launch_polynorm<bf16, float>(in, bias, coef, out, n_rows, cols, in_stride, eps, stream);
  if (act_dtype == IE_BF16 && w_dtype == IE_BF16)
    return launch_polynorm<bf16, bf16>(in, bias, coef, out, n_rows, cols, in_stride, eps, stream);
  return IE_BAD_DTYPE;
}

// ------------------------------------------ per-head RMS norm of q and k + cache write
// For token n: every query head and every key head is divided by its root mean square over the head
// (sqrt(mean(x^2) + eps)) and multiplied by a gain of the head's size that all heads share (a null gain
// leaves that side as it is).  q is normalised in place.  With `write_kv` the normalised k and the raw v go to
// the page slot slot_mapping[n] of pools laid out [page, kv_head, page_size, head size], where keys have `hd`
// and values `hd_v` elements a head, and a negative slot writes nothing; without it k is normalised in place
// (for whatever writes the cache afterwards).  One warp works on one head at a time.
template <typename TA, typename TW>
__global__ void headnorm_kv_write_kernel(TA* __restrict__ q, TA* __restrict__ k, const TA* __restrict__ v,
                                         int q_stride, int k_stride, int v_stride, const TW* __restrict__ q_gain,
                                         const TW* __restrict__ k_gain, float eps,
                                         const int* __restrict__ slot_mapping, TA* __restrict__ kpool,
                                         TA* __restrict__ vpool, int n_heads, int n_kv_heads, int hd, int hd_v,
                                         int page_size, int write_kv) {
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const int slot = write_kv ? IE_SLOT(slot_mapping[n]) : -1;
  const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot - page * page_size : 0;
  for (int h = warp; h < n_heads + n_kv_heads; h += n_warps) {
    const bool is_q = h < n_heads;
    const int hk = h - n_heads;
    if (!is_q && write_kv && slot < 0) continue;
    const TW* gain = is_q ? q_gain : k_gain;
    TA* src = is_q ? q + (size_t)n * q_stride + h * hd : k + (size_t)n * k_stride + hk * hd;
    TA* dst = (is_q || !write_kv) ? src : kpool + (((size_t)page * n_kv_heads + hk) * page_size + off) * hd;
    if (gain == nullptr) {
      if (dst != src)
        for (int i = lane; i < hd; i += 32) dst[i] = src[i];
      continue;
    }
    float ss = 0.f;
    for (int i = lane; i < hd; i += 32) {
      const float x = to_f32(src[i]);
      ss += x * x;
    }
    const float rms = sqrtf(warp_sum(ss) / (float)hd + eps);
    for (int i = lane; i < hd; i += 32) dst[i] = from_f32<TA>(to_f32(src[i]) / rms * to_f32(gain[i]));
  }
  if (slot < 0) return;
  const TA* vrow = v + (size_t)n * v_stride;
  for (int idx = threadIdx.x; idx < n_kv_heads * hd_v; idx += blockDim.x) {
    const int h = idx / hd_v, i = idx - h * hd_v;
    vpool[(((size_t)page * n_kv_heads + h) * page_size + off) * hd_v + i] = vrow[idx];
  }
}

template <typename TA, typename TW>
static int launch_headnorm(void* q, void* k, const void* v, int q_stride, int k_stride, int v_stride,
                           const void* q_gain, const void* k_gain, float eps, const int* slot_mapping, void* kpool,
                           void* vpool, int n_tokens, int n_heads, int n_kv_heads, int hd, int hd_v, int page_size,
                           int write_kv, cudaStream_t stream) {
  const int heads = n_heads + n_kv_heads;
  const int threads = heads >= 8 ? 256 : (heads >= 4 ? 128 : 64);
  return launch_k(headnorm_kv_write_kernel<TA, TW>, n_tokens, threads, 0, stream, (TA*)q, (TA*)k, (const TA*)v,
                  q_stride, k_stride, v_stride, (const TW*)q_gain, (const TW*)k_gain, eps, slot_mapping, (TA*)kpool,
                  (TA*)vpool, n_heads, n_kv_heads, hd, hd_v, page_size, write_kv);
}

extern "C" int ie_headnorm_kv_write(void* q, void* k, const void* v, int q_stride, int k_stride, int v_stride,
                                    const void* q_gain, const void* k_gain, int gain_dtype, float eps,
                                    const int* slot_mapping, void* kpool, void* vpool, int n_tokens, int n_heads,
                                    int n_kv_heads, int hd, int hd_v, int page_size, int write_kv, int act_dtype,
                                    cudaStream_t stream) {
  if (n_tokens <= 0) return IE_OK;
  if (hd <= 0 || hd_v <= 0) return IE_BAD_SIZE;
#define IE_HN(TA, TW)                                                                                              \
  return launch_headnorm<TA, TW>(q, k, v, q_stride, k_stride, v_stride, q_gain, k_gain, eps, slot_mapping, kpool, \
                                 vpool, n_tokens, n_heads, n_kv_heads, hd, hd_v, page_size, write_kv, stream)
  if (act_dtype == IE_F32 && gain_dtype == IE_F32) IE_HN(float, float);
  if (act_dtype == IE_F32 && gain_dtype == IE_BF16) IE_HN(float, bf16);
  if (act_dtype == IE_BF16 && gain_dtype == IE_F32) IE_HN(bf16, float);
  if (act_dtype == IE_BF16 && gain_dtype == IE_BF16) IE_HN(bf16, bf16);
#undef IE_HN
  return IE_BAD_DTYPE;
}

IE_CHECK_API(rowwise)
