// The gated delta rule: a recurrent mixer whose state is one DK x DV float32 matrix per (request, head).
//
// Per token and head, with the head's query q and key k (DK numbers; several heads may share one q/k head), its
// value v (DV numbers), a write strength beta = sigmoid(b_pre) and a decay g = exp(-exp(A_log) * softplus(a_pre +
// dt_bias)), both one number a head:
//     q <- q / sqrt(sum(q^2) + key_eps) * DK^-1/2,   k <- k / sqrt(sum(k^2) + key_eps)
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (o sees the token's own write)
// The head's o is divided by its root mean square over DV (norm_eps inside the root), multiplied by a gain of DV
// numbers that the heads share and by silu(gate), and written in the activation type for the output projection.
// Everything between the projections (q, k, v after their convolutions, b_pre, a_pre, gate) and that store is float32.
//
// DK and DV are compile-time constants (-DIE_GD_DK, -DIE_GD_DV): a library is built per pair when a model first asks.
// A block owns one (request, head).  Column j of S (value channel j) belongs to KS neighbouring threads, each with
// DK / KS of its rows in registers, so S^T k, the update and S^T q are sums inside a thread and a shuffle among
// those lanes.  The step's tokens of the request are walked in tiles of TT, whose q, k, v and gate are fetched into
// registers while the tile before is being run: (A) they go to shared memory as float32, a thread per token forms
// beta and g and a warp per token makes q and k unit vectors;
// (B) every thread runs the tile's tokens in order; (C) a warp per token norms and gates the outputs.  The order
// of every sum is fixed by the token and the channel alone, so a token's result does not depend on how the
// sequence was cut into steps or on what else the step holds.  A decode step is a tile of one token.
#include "common.cuh"

#if !defined(IE_GD_DK) || !defined(IE_GD_DV)
#error "gated_delta.cu is compiled per head size: -DIE_GD_DK=<key size> -DIE_GD_DV=<value size>"
#endif
#define GD_DK IE_GD_DK
#define GD_DV IE_GD_DV

constexpr int gd_pick_ks() {
  // the fewest lanes a column (1, 2, 4, 8) that leave a thread at most 32 rows; DK must split evenly
  for (int ks = 1; ks <= 8; ks *= 2)
    if (GD_DK % ks == 0 && GD_DK / ks <= 32 && GD_DV * ks <= 1024) return ks;
  for (int ks = 8; ks >= 1; ks /= 2)
    if (GD_DK % ks == 0 && GD_DV * ks <= 1024) return ks;
  return 1;
}
#define GD_KS (gd_pick_ks())
#define GD_DKP (GD_DK / GD_KS)                      // rows of a column in one thread
#define GD_THREADS (((GD_DV * GD_KS + 31) / 32) * 32)
#define GD_TT ((2 * GD_DK + 3 * GD_DV) <= 640 ? 16 : 8)
// the q and k vectors lie in shared memory part by part, each part GD_LD floats after the one before: the padding
// puts the parts that the KS lanes of a column read at once on different banks
#define GD_LD (GD_DKP + (GD_KS > 1 ? 4 : 0))
#define GD_ROW (GD_KS * GD_LD)
#define GD_VEC (GD_DKP % 4 == 0)

static_assert(GD_DK >= 1 && GD_DV >= 1 && GD_DV <= 1024, "value heads up to 1024 channels: one block a head");
static_assert(GD_DKP <= 128, "a thread keeps its rows of a state column in registers");
static_assert(GD_TT * (2 * GD_ROW + 3 * GD_DV + 3) * 4 <= 48 * 1024, "a tile's vectors must fit in shared memory");

struct GatedDeltaParams {
  const void* q;            // activation type, [N, *_stride]: columns of one buffer (after convolution and SiLU)
  const void* k;
  const void* v;
  int qk_stride, v_stride;
  const void* b_pre;        // activation type [N, ba_stride], one column a head
  const void* a_pre;
  int ba_stride;
  const void* gate;         // activation type [N, gate_stride], heads x DV
  int gate_stride;
  const void* a_log;        // weight type [H]
  const void* dt_bias;      // weight type [H]
  const void* out_gain;     // weight type [DV]
  float* state;             // [slots, H, DK, DV] float32
  void* out;                // activation type [N, out_stride]
  int out_stride;
  const int* q_start;       // [R + 1]
  const int* slots;         // [R], negative: a padding row without state
  int n_heads, n_kv_heads;
  float key_eps, norm_eps;
  int write_state;
};

// Loads of a tile's inputs that stay where they are written (volatile): they are issued before the tile ahead is run
// and used after it; left to itself the compiler moves them down to their use and the tile then waits for memory.
__device__ __forceinline__ float gd_ld_early(const float* p) {
  float v;
  asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ float gd_ld_early(const bf16* p) {
  unsigned short v;
  asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return __uint_as_float((unsigned)v << 16);
}
#define GD_PQ ((GD_TT * GD_DK + GD_THREADS - 1) / GD_THREADS)   // elements of a tile's q (and k) a thread fetches
#define GD_PV ((GD_TT * GD_DV + GD_THREADS - 1) / GD_THREADS)   // of its v (and gate)

__device__ __forceinline__ int gd_place(int i) { return (i / GD_DKP) * GD_LD + (i % GD_DKP); }   // channel -> place
__device__ __forceinline__ float gd_column_sum(float v) {
#pragma unroll
  for (int o = 1; o < GD_KS; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename TA, typename TW>
__global__ void __launch_bounds__(GD_THREADS) gated_delta_kernel(GatedDeltaParams p) {
  __shared__ __align__(16) float sq[GD_TT][GD_ROW], sk[GD_TT][GD_ROW];
  __shared__ float sv[GD_TT][GD_DV], sg[GD_TT][GD_DV], so[GD_TT][GD_DV], sbeta[GD_TT], sdecay[GD_TT], sdecm1[GD_TT];
  pdl_trigger();
  pdl_wait();
  const int req = blockIdx.x, h = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int n_warps = GD_THREADS / 32;
  const int j = tid / GD_KS, part = tid - j * GD_KS;
  const bool active = j < GD_DV;
  const int row0 = part * GD_DKP, base = part * GD_LD;
  const int q0 = p.q_start[req], q1 = p.q_start[req + 1];
  const int slot = IE_SLOT(p.slots[req]);
  const int c = h / (p.n_heads / p.n_kv_heads);         // the q/k head this head reads
  TA* out = (TA*)p.out;
  if (slot < 0) {
    for (int idx = tid; idx < (q1 - q0) * GD_DV; idx += GD_THREADS)
      out[(size_t)(q0 + idx / GD_DV) * p.out_stride + h * GD_DV + idx % GD_DV] = from_f32<TA>(0.f);
    return;
  }
  const TA* Q = (const TA*)p.q + c * GD_DK;
  const TA* K = (const TA*)p.k + c * GD_DK;
  const TA* V = (const TA*)p.v + h * GD_DV;
  const TA* G = (const TA*)p.gate + h * GD_DV;
  const float rate = -expf(to_f32(((const TW*)p.a_log)[h]));
  const float dt_bias = to_f32(((const TW*)p.dt_bias)[h]);
  const TW* gain = (const TW*)p.out_gain;
  const float q_scale = rsqrtf((float)GD_DK);

  float S[GD_DKP];
  float* st = p.state + (((size_t)slot * p.n_heads + h) * GD_DK) * GD_DV;
#pragma unroll
  for (int i = 0; i < GD_DKP; ++i) S[i] = active ? st[(size_t)(row0 + i) * GD_DV + j] : 0.f;

  // a tile's inputs in registers, fetched while the tile ahead is being run
  float fq[GD_PQ], fk[GD_PQ], fv[GD_PV], fg[GD_PV];
  auto fetch = [&](int t0, int nt) {
#pragma unroll
    for (int u = 0; u < GD_PQ; ++u) {
      const int e = tid + u * GD_THREADS;
      const int tt = e / GD_DK, i = e - tt * GD_DK;
      if (tt < nt) {
        const size_t row = (size_t)(t0 + tt) * p.qk_stride + i;
        fq[u] = gd_ld_early(Q + row);
        fk[u] = gd_ld_early(K + row);
      }
    }
#pragma unroll
    for (int u = 0; u < GD_PV; ++u) {
      const int e = tid + u * GD_THREADS;
      const int tt = e / GD_DV, i = e - tt * GD_DV;
      if (tt < nt) {
        fv[u] = gd_ld_early(V + (size_t)(t0 + tt) * p.v_stride + i);
        fg[u] = gd_ld_early(G + (size_t)(t0 + tt) * p.gate_stride + i);
      }
    }
  };
  if (q0 < q1) fetch(q0, min(GD_TT, q1 - q0));

  for (int t0 = q0; t0 < q1; t0 += GD_TT) {
    const int nt = min(GD_TT, q1 - t0);
    // (A) the tile's vectors, the two numbers of every token, the unit vectors
#pragma unroll
    for (int u = 0; u < GD_PQ; ++u) {
      const int e = tid + u * GD_THREADS;
      const int tt = e / GD_DK, i = e - tt * GD_DK;
      if (tt < nt) {
        sq[tt][gd_place(i)] = fq[u];
        sk[tt][gd_place(i)] = fk[u];
      }
    }
#pragma unroll
    for (int u = 0; u < GD_PV; ++u) {
      const int e = tid + u * GD_THREADS;
      const int tt = e / GD_DV, i = e - tt * GD_DV;
      if (tt < nt) {
        sv[tt][i] = fv[u];
        sg[tt][i] = to_f32(gain[i]) * (fg[u] / (1.f + expf(-fg[u])));
      }
    }
    if (tid < nt) {
      const float b = to_f32(((const TA*)p.b_pre)[(size_t)(t0 + tid) * p.ba_stride + h]);
      const float a = to_f32(((const TA*)p.a_pre)[(size_t)(t0 + tid) * p.ba_stride + h]) + dt_bias;
      sbeta[tid] = 1.f / (1.f + expf(-b));
      // the decay, and the decay less one when it is above one half: a float32 decay of 1 - 2.5e-6 is off by up to a
      // hundredth of its distance from one, which a thousand tokens turn into the fifth digit of the state
      const float log_g = rate * (a > 20.f ? a : log1pf(expf(a)));
      sdecay[tid] = expf(log_g);
      sdecm1[tid] = log_g > -0.6931472f ? expm1f(log_g) : 0.f;
    }
    __syncthreads();
    for (int tt = warp; tt < nt; tt += n_warps) {
      float qq = 0.f, kk = 0.f;
      for (int i = lane; i < GD_DK; i += 32) {
        const float a = sq[tt][gd_place(i)], b = sk[tt][gd_place(i)];
        qq = fmaf(a, a, qq);
        kk = fmaf(b, b, kk);
      }
      const float qn = q_scale / sqrtf(warp_sum(qq) + p.key_eps), kn = 1.f / sqrtf(warp_sum(kk) + p.key_eps);
      for (int i = lane; i < GD_DK; i += 32) {
        sq[tt][gd_place(i)] *= qn;
        sk[tt][gd_place(i)] *= kn;
      }
    }
    __syncthreads();
    if (t0 + GD_TT < q1) fetch(t0 + GD_TT, min(GD_TT, q1 - t0 - GD_TT));     // lands while this tile runs
    // (B) the tile's tokens in order; this thread's rows of its column of the state
#pragma unroll 2
    for (int tt = 0; tt < nt; ++tt) {
      float kk[GD_DKP], qq[GD_DKP];
      if constexpr (GD_VEC) {
#pragma unroll
        for (int i = 0; i < GD_DKP; i += 4) {
          *reinterpret_cast<float4*>(&kk[i]) = *reinterpret_cast<const float4*>(&sk[tt][base + i]);
          *reinterpret_cast<float4*>(&qq[i]) = *reinterpret_cast<const float4*>(&sq[tt][base + i]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < GD_DKP; ++i) {
          kk[i] = sk[tt][base + i];
          qq[i] = sq[tt][base + i];
        }
      }
      const float vj = active ? sv[tt][j] : 0.f;
      const float g = sdecay[tt], gm1 = sdecm1[tt], beta = sbeta[tt];
      float ks[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < GD_DKP; ++i) ks[i & 3] = fmaf(kk[i], S[i], ks[i & 3]);
      const float sk_old = gd_column_sum((ks[0] + ks[1]) + (ks[2] + ks[3]));
      float u;
      if (gm1 != 0.f) {                  // g S as S + (g - 1) S
        u = beta * (vj - fmaf(gm1, sk_old, sk_old));                                // (g S)^T k
#pragma unroll
        for (int i = 0; i < GD_DKP; ++i) S[i] = fmaf(kk[i], u, fmaf(gm1, S[i], S[i]));
      } else {
        u = beta * (vj - g * sk_old);
#pragma unroll
        for (int i = 0; i < GD_DKP; ++i) S[i] = fmaf(kk[i], u, g * S[i]);
      }
      float oo[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < GD_DKP; ++i) oo[i & 3] = fmaf(S[i], qq[i], oo[i & 3]);
      const float o = gd_column_sum((oo[0] + oo[1]) + (oo[2] + oo[3]));
      if (active && part == 0) so[tt][j] = o;
    }
    __syncthreads();
    // (C) norm over the head, gain, gate; a warp per token
    for (int tt = warp; tt < nt; tt += n_warps) {
      float ss = 0.f;
      for (int i = lane; i < GD_DV; i += 32) ss = fmaf(so[tt][i], so[tt][i], ss);
      const float rms = sqrtf(warp_sum(ss) / (float)GD_DV + p.norm_eps);
      for (int i = lane; i < GD_DV; i += 32)
        out[(size_t)(t0 + tt) * p.out_stride + h * GD_DV + i] = from_f32<TA>(so[tt][i] / rms * sg[tt][i]);
    }
    __syncthreads();
  }
  if (p.write_state && active) {
#pragma unroll
    for (int i = 0; i < GD_DKP; ++i) st[(size_t)(row0 + i) * GD_DV + j] = S[i];
  }
}

extern "C" int ie_gated_delta_dims(int* dk, int* dv) {
  *dk = GD_DK;
  *dv = GD_DV;
  return IE_OK;
}

extern "C" int ie_gated_delta(const void* q, const void* k, const void* v, int qk_stride, int v_stride,
                              const void* b_pre, const void* a_pre, int ba_stride, const void* gate, int gate_stride,
                              const void* a_log, const void* dt_bias, const void* out_gain, int w_dtype, float* state,
                              void* out, int out_stride, const int* q_start, const int* slots, int n_requests,
                              int n_heads, int n_kv_heads, int dk, int dv, float key_eps, float norm_eps,
                              int write_state, int act_dtype, cudaStream_t stream) {
  if (n_requests <= 0 || n_heads <= 0) return IE_OK;
  if (dk != GD_DK || dv != GD_DV || n_kv_heads <= 0 || n_heads % n_kv_heads) return IE_BAD_SIZE;
  GatedDeltaParams p;
  p.q = q; p.k = k; p.v = v; p.qk_stride = qk_stride; p.v_stride = v_stride; p.b_pre = b_pre; p.a_pre = a_pre;
  p.ba_stride = ba_stride; p.gate = gate; p.gate_stride = gate_stride; p.a_log = a_log; p.dt_bias = dt_bias;
  p.out_gain = out_gain; p.state = state; p.out = out; p.out_stride = out_stride; p.q_start = q_start; p.slots = slots;
  p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.key_eps = key_eps; p.norm_eps = norm_eps; p.write_state = write_state;
  dim3 grid(n_requests, n_heads);
  if (act_dtype == IE_F32 && w_dtype == IE_F32) return launch_k(gated_delta_kernel<float, float>, grid, GD_THREADS, 0, stream, p);
  if (act_dtype == IE_F32 && w_dtype == IE_BF16) return launch_k(gated_delta_kernel<float, bf16>, grid, GD_THREADS, 0, stream, p);
  if (act_dtype == IE_BF16 && w_dtype == IE_F32) return launch_k(gated_delta_kernel<bf16, float>, grid, GD_THREADS, 0, stream, p);
  if (act_dtype == IE_BF16 && w_dtype == IE_BF16) return launch_k(gated_delta_kernel<bf16, bf16>, grid, GD_THREADS, 0, stream, p);
  return IE_BAD_DTYPE;
}

IE_CHECK_API(gated_delta)
