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
  if (smem > 47 * 1024) {      // the static reduction scratch counts towards the 48 KB that need no opt-in
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

// eight bfloat16 (16 bytes) as float32
__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const float2 x = __bfloat1622float2(h[t]);
    f[2 * t] = x.x;
    f[2 * t + 1] = x.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int t = 0; t < 4; ++t) h[t] = __floats2bfloat162_rn(f[2 * t], f[2 * t + 1]);
  return raw;
}

// the same for bfloat16 tables whose rows are a multiple of eight wide: 16 bytes a load, 32 a store
__global__ void embed_bigram_bf16_vec_kernel(const int* __restrict__ ids, const int* __restrict__ positions,
                                             const int* __restrict__ q_start, const int* __restrict__ slots,
                                             int n_requests, const bf16* __restrict__ table,
                                             const bf16* __restrict__ bigram, int* __restrict__ prev_state,
                                             float* __restrict__ residual, int d, int vocab, int buckets,
                                             long long mul_prev, long long mul_cur) {
  __shared__ int s_row, s_id;
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  if (threadIdx.x == 0) {
    int lo = 0, hi = n_requests;
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
      if (hsh < 0) hsh += buckets;
      row = (int)hsh;
    }
    if (n == first && slot >= 0) prev_state[slot] = ids[q_start[r + 1] - 1];
    s_row = row;
    s_id = id;
  }
  __syncthreads();
  const bf16* a = table + (size_t)s_id * d;
  const bf16* b = bigram + (size_t)s_row * d;
  float* out = residual + (size_t)n * d;
  for (int i = threadIdx.x * 8; i < d; i += blockDim.x * 8) {
    float x[8], y[8];
    unpack8(*reinterpret_cast<const uint4*>(a + i), x);
    unpack8(*reinterpret_cast<const uint4*>(b + i), y);
    *reinterpret_cast<float4*>(out + i) = make_float4(x[0] + y[0], x[1] + y[1], x[2] + y[2], x[3] + y[3]);
    *reinterpret_cast<float4*>(out + i + 4) = make_float4(x[4] + y[4], x[5] + y[5], x[6] + y[6], x[7] + y[7]);
  }
}

extern "C" int ie_embed_bigram(const int* ids, const int* positions, const int* q_start, const int* slots,
                               int n_requests, const void* table, const void* bigram, int table_dtype,
                               int* prev_state, float* residual, int n_tokens, int d, int vocab, int buckets,
                               long long mul_prev, long long mul_cur, cudaStream_t stream) {
  if (n_tokens <= 0) return IE_OK;
  if (buckets <= 0 || n_requests <= 0) return IE_BAD_SIZE;
  const int threads = d >= 1024 ? 256 : 128;
  if (table_dtype == IE_BF16 && d % 8 == 0 && (((uintptr_t)table | (uintptr_t)bigram | (uintptr_t)residual) & 15) == 0)
    return launch_k(embed_bigram_bf16_vec_kernel, n_tokens, d >= 2048 ? 256 : 128, 0, stream, ids, positions, q_start,
                    slots, n_requests, (const bf16*)table, (const bf16*)bigram, prev_state, residual, d, vocab, buckets,
                    mul_prev, mul_cur);
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

// Three sums over a block at once, in a fixed order (warp trees, then the warps in order); `scratch` holds 99 floats.
__device__ __forceinline__ void block_sum3(float& a, float& b, float& c, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_warps = (blockDim.x + 31) >> 5;
  a = warp_sum(a);
  b = warp_sum(b);
  c = warp_sum(c);
  if (lane == 0) {
    scratch[warp] = a;
    scratch[33 + warp] = b;
    scratch[66 + warp] = c;
  }
  __syncthreads();
  float ta = 0.f, tb = 0.f, tc = 0.f;
  for (int w = 0; w < n_warps; ++w) {      // every thread adds the warps up in the same order
    ta += scratch[w];
    tb += scratch[33 + w];
    tc += scratch[66 + w];
  }
  a = ta; b = tb; c = tc;
}

// bfloat16 rows whose width is a multiple of eight: 16 bytes a load and a store, the row staged as float4;
// one reduction for the three sums, and the three divisions of an element become products with the row's
// reciprocals (the result is rounded to bfloat16 right after)
__global__ void polynorm_bf16_vec_kernel(const bf16* __restrict__ in, const bf16* __restrict__ bias,
                                         const bf16* __restrict__ coef, bf16* __restrict__ out, int cols, int in_stride,
                                         float eps) {
  extern __shared__ __align__(16) float zs[];
  __shared__ float red[99];
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  const bf16* row = in + (size_t)n * in_stride;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int i = threadIdx.x * 8; i < cols; i += blockDim.x * 8) {
    float z[8];
    unpack8(*reinterpret_cast<const uint4*>(row + i), z);
    if (bias) {
      float b[8];
      unpack8(*reinterpret_cast<const uint4*>(bias + i), b);
#pragma unroll
      for (int t = 0; t < 8; ++t) z[t] += b[t];
    }
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const float z2 = z[t] * z[t], z3 = z2 * z[t];
      s2 += z2;
      s4 += z2 * z2;
      s6 += z3 * z3;
    }
    *reinterpret_cast<float4*>(zs + i) = make_float4(z[0], z[1], z[2], z[3]);
    *reinterpret_cast<float4*>(zs + i + 4) = make_float4(z[4], z[5], z[6], z[7]);
  }
  block_sum3(s2, s4, s6, red);
  const float c3 = to_f32(coef[3]);
  const float k1 = to_f32(coef[0]) / sqrtf(s2 / (float)cols + eps);
  const float k2 = to_f32(coef[1]) / sqrtf(s4 / (float)cols + eps);
  const float k3 = to_f32(coef[2]) / sqrtf(s6 / (float)cols + eps);
  bf16* o = out + (size_t)n * cols;
  for (int i = threadIdx.x * 8; i < cols; i += blockDim.x * 8) {       // a thread reads back what it wrote itself
    const float4 a = *reinterpret_cast<const float4*>(zs + i), b = *reinterpret_cast<const float4*>(zs + i + 4);
    const float z[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float y[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const float z2 = z[t] * z[t];
      y[t] = fmaf(k1, z[t], fmaf(k2, z2, fmaf(k3, z2 * z[t], c3)));
    }
    *reinterpret_cast<uint4*>(o + i) = pack8(y);
  }
}

template <typename TA, typename TW>
static int launch_polynorm(const void* in, const void* bias, const void* coef, void* out, int n_rows, int cols,
                           int in_stride, float eps, cudaStream_t stream) {
  const size_t smem = (size_t)cols * sizeof(float);
  if (smem > 200 * 1024) return IE_BAD_SIZE;
  if (smem > 47 * 1024) {      // the static reduction scratch counts towards the 48 KB that need no opt-in
    cudaError_t e = cudaFuncSetAttribute(polynorm_kernel<TA, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int threads = cols >= 4096 ? 512 : (cols >= 512 ? 256 : 128);
  if (sizeof(TA) == 2 && sizeof(TW) == 2 && cols % 8 == 0 && in_stride % 8 == 0 &&
      (((uintptr_t)in | (uintptr_t)bias | (uintptr_t)out) & 15) == 0) {
    if (smem > 47 * 1024) {      // the static reduction scratch counts towards the 48 KB that need no opt-in
      cudaError_t e = cudaFuncSetAttribute(polynorm_bf16_vec_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    return launch_k(polynorm_bf16_vec_kernel, n_rows, cols >= 4096 ? 256 : 128, smem, stream, (const bf16*)in,
                    (const bf16*)bias, (const bf16*)coef, (bf16*)out, cols, in_stride, eps);
  }
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

// bfloat16 activations and gains, head sizes that are multiples of eight up to 256: a lane holds eight elements of
// a head (16 bytes), so a head is one load, one sum over the warp and one store; values are copied 16 bytes a lane
__global__ void headnorm_kv_write_bf16_vec_kernel(bf16* __restrict__ q, bf16* __restrict__ k, const bf16* __restrict__ v,
                                                  int q_stride, int k_stride, int v_stride,
                                                  const bf16* __restrict__ q_gain, const bf16* __restrict__ k_gain,
                                                  float eps, const int* __restrict__ slot_mapping,
                                                  bf16* __restrict__ kpool, bf16* __restrict__ vpool, int n_heads,
                                                  int n_kv_heads, int hd, int hd_v, int page_size, int write_kv) {
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const int slot = write_kv ? IE_SLOT(slot_mapping[n]) : -1;
  const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot - page * page_size : 0;
  const bool mine = lane * 8 < hd;
  for (int h = warp; h < n_heads + n_kv_heads; h += n_warps) {
    const bool is_q = h < n_heads;
    const int hk = h - n_heads;
    if (!is_q && write_kv && slot < 0) continue;
    const bf16* gain = is_q ? q_gain : k_gain;
    bf16* src = is_q ? q + (size_t)n * q_stride + h * hd : k + (size_t)n * k_stride + hk * hd;
    bf16* dst = (is_q || !write_kv) ? src : kpool + (((size_t)page * n_kv_heads + hk) * page_size + off) * hd;
    if (gain == nullptr && dst == src) continue;
    float x[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (mine) {
      raw = *reinterpret_cast<const uint4*>(src + lane * 8);
      unpack8(raw, x);
    }
    if (gain == nullptr) {
      if (mine) *reinterpret_cast<uint4*>(dst + lane * 8) = raw;
      continue;
    }
    float ss = 0.f;
#pragma unroll
    for (int t = 0; t < 8; ++t) ss += x[t] * x[t];
    const float rms = sqrtf(warp_sum(ss) / (float)hd + eps);
    if (mine) {
      float g[8];
      unpack8(*reinterpret_cast<const uint4*>(gain + lane * 8), g);
#pragma unroll
      for (int t = 0; t < 8; ++t) x[t] = x[t] / rms * g[t];
      *reinterpret_cast<uint4*>(dst + lane * 8) = pack8(x);
    }
  }
  if (slot < 0) return;
  const bf16* vrow = v + (size_t)n * v_stride;
  const int per_head = hd_v >> 3;
  for (int idx = threadIdx.x; idx < n_kv_heads * per_head; idx += blockDim.x) {
    const int h = idx / per_head, i = (idx - h * per_head) * 8;
    *reinterpret_cast<uint4*>(vpool + (((size_t)page * n_kv_heads + h) * page_size + off) * hd_v + i) =
        *reinterpret_cast<const uint4*>(vrow + h * hd_v + i);
  }
}

template <typename TA, typename TW>
static int launch_headnorm(void* q, void* k, const void* v, int q_stride, int k_stride, int v_stride,
                           const void* q_gain, const void* k_gain, float eps, const int* slot_mapping, void* kpool,
                           void* vpool, int n_tokens, int n_heads, int n_kv_heads, int hd, int hd_v, int page_size,
                           int write_kv, cudaStream_t stream) {
  const int heads = n_heads + n_kv_heads;
  const int threads = heads >= 8 ? 256 : (heads >= 4 ? 128 : 64);
  if (sizeof(TA) == 2 && sizeof(TW) == 2 && hd % 8 == 0 && hd <= 256 && hd_v % 8 == 0 && q_stride % 8 == 0 &&
      k_stride % 8 == 0 && v_stride % 8 == 0 &&
      (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)q_gain | (uintptr_t)k_gain | (uintptr_t)kpool |
        (uintptr_t)vpool) & 15) == 0)
    return launch_k(headnorm_kv_write_bf16_vec_kernel, n_tokens, threads, 0, stream, (bf16*)q, (bf16*)k, (const bf16*)v,
                    q_stride, k_stride, v_stride, (const bf16*)q_gain, (const bf16*)k_gain, eps, slot_mapping,
                    (bf16*)kpool, (bf16*)vpool, n_heads, n_kv_heads, hd, hd_v, page_size, write_kv);
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
