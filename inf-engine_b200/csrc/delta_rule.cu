// The generalized delta rule: a recurrent mixer whose state is one D x D float32 matrix per (request, head).
//
// For a token with receptance r, key k, value v (D numbers each a head), a decay w and a removal rate a per
// key channel, and the unit key u = k / sqrt(sum(k^2) + key_eps):
//     S <- diag(w) S - (a * u) (u^T S) + k v^T          (both terms read the old state)
//     o  = S^T r
// with  w = exp(-decay_rate * sigmoid(w_pre + w_bias)),  a = sigmoid(a_pre + a_bias),  w_pre and a_pre being
// projections of the token.  The head's o is divided by its root mean square (norm_eps inside the root),
// multiplied by a gain over all heads and by sigmoid(g), and written in the activation type for the output
// projection.  Everything between the projections and that last store is float32.
//
// The head size D is a compile-time constant (-DIE_DR_DIM): a library is built per size when a model first asks.
// A block owns one (request, head) and has one thread per value column: thread j keeps column j of S (D
// registers).  With that layout u^T S, the update and S^T r are sums inside a thread; nothing crosses threads
// but the two norms.  The step's tokens of the request are walked in tiles: (A) the warps prepare the tile's
// k, r, w, a*u and u in shared memory, a warp per token; (B) every thread runs the tile's tokens in order,
// reading those vectors as broadcasts; (C) the warps norm and gate the tile's outputs, a warp per token.
// The order of every sum is fixed by the token and the channel alone, so a token's result does not depend on
// how the sequence was cut into steps or on what else the step holds.  A decode step is a tile of one token.
#include "common.cuh"

#ifndef IE_DR_DIM
#error "delta_rule.cu is compiled per head size: -DIE_DR_DIM=<size>"
#endif
#define DR_D IE_DR_DIM
#define DR_TT (DR_D > 64 ? 8 : 16)                 // tokens a tile
#define DR_THREADS (((DR_D + 31) / 32) * 32)

static_assert(DR_D >= 1 && DR_D <= 128, "head sizes up to 128: a thread keeps a column of the state in registers");

struct DeltaRuleParams {
  const void* r;            // activation type, [N, stride]: columns of one projection buffer
  const void* k;
  const void* v;
  const void* a_pre;
  const void* g;
  int stride;
  const float* w_pre;       // float32 [N, w_stride]
  int w_stride;
  const void* a_bias;       // weight type, [H * D]
  const void* w_bias;
  const void* out_gain;
  float* state;             // [slots, H, D, D] float32; row = key channel, column = value channel
  void* out;                // activation type, [N, out_stride]
  int out_stride;
  const int* q_start;       // [R + 1]
  const int* slots;         // [R], negative: a padding row without state
  int n_heads;
  float decay_rate, key_eps, norm_eps;
  int write_state;
};

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }

template <typename TA, typename TW>
__global__ void __launch_bounds__(DR_THREADS) delta_rule_kernel(DeltaRuleParams p) {
  __shared__ __align__(16) float sk[DR_TT][DR_D], sr[DR_TT][DR_D], sw[DR_TT][DR_D], sb[DR_TT][DR_D], su[DR_TT][DR_D],
      so[DR_TT][DR_D];
  pdl_trigger();
  pdl_wait();
  const int req = blockIdx.x, h = blockIdx.y;
  const int j = threadIdx.x;
  const int lane = j & 31, warp = j >> 5;
  constexpr int n_warps = DR_THREADS / 32;
  const int q0 = p.q_start[req], q1 = p.q_start[req + 1];
  const int slot = IE_SLOT(p.slots[req]);
  const int col0 = h * DR_D;
  TA* out = (TA*)p.out;
  if (slot < 0) {
    for (int n = q0; n < q1; ++n)
      if (j < DR_D) out[(size_t)n * p.out_stride + col0 + j] = from_f32<TA>(0.f);
    return;
  }
  const TA* R = (const TA*)p.r;
  const TA* K = (const TA*)p.k;
  const TA* V = (const TA*)p.v;
  const TA* A = (const TA*)p.a_pre;
  const TA* G = (const TA*)p.g;
  const TW* a_bias = (const TW*)p.a_bias;
  const TW* w_bias = (const TW*)p.w_bias;
  const TW* gain = (const TW*)p.out_gain;

  float S[DR_D];
  float* st = p.state + (((size_t)slot * p.n_heads + h) * DR_D) * DR_D;
  if (j < DR_D) {
#pragma unroll
    for (int i = 0; i < DR_D; ++i) S[i] = st[(size_t)i * DR_D + j];
  }

  for (int t0 = q0; t0 < q1; t0 += DR_TT) {
    const int nt = min(DR_TT, q1 - t0);
    // (A) the tile's vectors, a warp per token
    for (int tt = warp; tt < nt; tt += n_warps) {
      const size_t row = (size_t)(t0 + tt) * p.stride + col0;
      const float* wp = p.w_pre + (size_t)(t0 + tt) * p.w_stride + col0;
      float ss = 0.f;
      for (int i = lane; i < DR_D; i += 32) {
        const float kk = to_f32(K[row + i]);
        ss += kk * kk;
      }
      const float knorm = sqrtf(warp_sum(ss) + p.key_eps);
      for (int i = lane; i < DR_D; i += 32) {
        const float kk = to_f32(K[row + i]);
        const float u = kk / knorm;
        const float a = sigmoidf_(to_f32(A[row + i]) + to_f32(a_bias[col0 + i]));
        const float w = expf(-p.decay_rate * sigmoidf_(wp[i] + to_f32(w_bias[col0 + i])));
        sk[tt][i] = kk;
        sr[tt][i] = to_f32(R[row + i]);
        sw[tt][i] = w;
        sb[tt][i] = a * u;
        su[tt][i] = u;
      }
    }
    float vv[DR_TT];
    if (j < DR_D) {
#pragma unroll
      for (int tt = 0; tt < DR_TT; ++tt) vv[tt] = tt < nt ? to_f32(V[(size_t)(t0 + tt) * p.stride + col0 + j]) : 0.f;
    }
    __syncthreads();
    // (B) the tile's tokens in order; this thread's column of the state
    if (j < DR_D) {
#pragma unroll
      for (int tt = 0; tt < DR_TT; ++tt) {
        if (tt < nt) {
          float us0 = 0.f, us1 = 0.f, us2 = 0.f, us3 = 0.f;
#pragma unroll
          for (int i = 0; i < DR_D; ++i) {
            const float t = su[tt][i] * S[i];
            if ((i & 3) == 0) us0 += t; else if ((i & 3) == 1) us1 += t; else if ((i & 3) == 2) us2 += t; else us3 += t;
          }
          const float us = (us0 + us1) + (us2 + us3);
          const float vj = vv[tt];
          float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
          for (int i = 0; i < DR_D; ++i) {
            const float add = fmaf(-sb[tt][i], us, sk[tt][i] * vj);
            S[i] = fmaf(sw[tt][i], S[i], add);
            const float t = S[i] * sr[tt][i];
            if ((i & 3) == 0) o0 += t; else if ((i & 3) == 1) o1 += t; else if ((i & 3) == 2) o2 += t; else o3 += t;
          }
          so[tt][j] = (o0 + o1) + (o2 + o3);
        }
      }
    }
    __syncthreads();
    // (C) norm over the head, gain, gate; a warp per token
    for (int tt = warp; tt < nt; tt += n_warps) {
      float ss = 0.f;
      for (int i = lane; i < DR_D; i += 32) ss += so[tt][i] * so[tt][i];
      const float rms = sqrtf(warp_sum(ss) / (float)DR_D + p.norm_eps);
      const size_t row = (size_t)(t0 + tt) * p.stride + col0;
      for (int i = lane; i < DR_D; i += 32) {
        const float y = so[tt][i] / rms * to_f32(gain[col0 + i]) * sigmoidf_(to_f32(G[row + i]));
        out[(size_t)(t0 + tt) * p.out_stride + col0 + i] = from_f32<TA>(y);
      }
    }
    __syncthreads();
  }
  if (p.write_state && j < DR_D) {
#pragma unroll
    for (int i = 0; i < DR_D; ++i) st[(size_t)i * DR_D + j] = S[i];
  }
}

extern "C" int ie_delta_rule_dim() { return DR_D; }

extern "C" int ie_delta_rule(const void* r, const void* k, const void* v, const void* a_pre, const void* g, int stride,
                             const float* w_pre, int w_stride, const void* a_bias, const void* w_bias,
                             const void* out_gain, int w_dtype, float* state, void* out, int out_stride,
                             const int* q_start, const int* slots, int n_requests, int n_heads, int head_dim,
                             float decay_rate, float key_eps, float norm_eps, int write_state, int act_dtype,
                             cudaStream_t stream) {
  if (n_requests <= 0 || n_heads <= 0) return IE_OK;
  if (head_dim != DR_D) return IE_BAD_SIZE;
  DeltaRuleParams p;
  p.r = r; p.k = k; p.v = v; p.a_pre = a_pre; p.g = g; p.stride = stride; p.w_pre = w_pre; p.w_stride = w_stride;
  p.a_bias = a_bias; p.w_bias = w_bias; p.out_gain = out_gain; p.state = state; p.out = out; p.out_stride = out_stride;
  p.q_start = q_start; p.slots = slots; p.n_heads = n_heads; p.decay_rate = decay_rate; p.key_eps = key_eps;
  p.norm_eps = norm_eps; p.write_state = write_state;
  dim3 grid(n_requests, n_heads);
  if (act_dtype == IE_F32 && w_dtype == IE_F32) return launch_k(delta_rule_kernel<float, float>, grid, DR_THREADS, 0, stream, p);
  if (act_dtype == IE_F32 && w_dtype == IE_BF16) return launch_k(delta_rule_kernel<float, bf16>, grid, DR_THREADS, 0, stream, p);
  if (act_dtype == IE_BF16 && w_dtype == IE_F32) return launch_k(delta_rule_kernel<bf16, float>, grid, DR_THREADS, 0, stream, p);
  if (act_dtype == IE_BF16 && w_dtype == IE_BF16) return launch_k(delta_rule_kernel<bf16, bf16>, grid, DR_THREADS, 0, stream, p);
  return IE_BAD_DTYPE;
}

IE_CHECK_API(delta_rule)
