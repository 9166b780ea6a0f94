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
// A block owns one (request, head).  A column of S (one value channel) belongs to KS neighbouring threads, each
// with D / KS of its rows in registers: u^T S, the update and S^T r are sums inside a thread and a shuffle
// among those KS lanes; nothing else crosses threads but the two norms.  The step's tokens of the request are
// walked in tiles of TT: the tile's six inputs are fetched into registers by all threads (one batch of
// independent loads, issued while the tile before is being run); then (A) they go to shared memory as k, r,
// decay, rate, gate * gain and v, and a warp per token turns k and rate into u and rate * u; (B) every thread
// runs the tile's tokens in order, reading those vectors as broadcasts; (C) a warp per token norms and gates
// the outputs.  The order of every sum is fixed by the token and the channel alone, so a token's result does
// not depend on how the sequence was cut into steps or on what else the step holds.  A decode step is a tile
// of one token.
#include "common.cuh"

#ifndef IE_DR_DIM
#error "delta_rule.cu is compiled per head size: -DIE_DR_DIM=<size>"
#endif
#define DR_D IE_DR_DIM
#define DR_TT (DR_D > 64 ? 8 : 16)                 // tokens a tile
#ifdef IE_DR_KS
#define DR_KS IE_DR_KS                             // threads a column (a build may say; measurements)
#else
// threads a column; measured on a B200 over a prompt of 2,048 tokens, 1,024 channels: heads of 64: 4, 2, 1 threads
// take 1.34, 1.45, 2.44 ms; heads of 128: 3.56, 2.50, 3.36 ms
#define DR_KS (DR_D > 64 ? (DR_D % 2 == 0 ? 2 : 1) : ((DR_D % 4 == 0 && DR_D > 32) ? 4 : ((DR_D % 2 == 0 && DR_D > 16) ? 2 : 1)))
#endif
#define DR_DK (DR_D / DR_KS)                       // rows of a column in one thread
#define DR_THREADS (((DR_D * DR_KS + 31) / 32) * 32)
#define DR_PER ((DR_TT * DR_D + DR_THREADS - 1) / DR_THREADS)   // elements of a tile's input a thread fetches
// The vectors that the KS threads of a column read by rows lie in shared memory part by part, each part DR_LD
// floats after the one before: the four floats of padding put the parts on different banks, so that one 16-byte
// load of a warp (KS different addresses) is served at once.
#define DR_LD (DR_DK + (DR_KS > 1 ? 4 : 0))
#define DR_ROW (DR_KS * DR_LD)
#define DR_VEC (DR_DK % 4 == 0)

static_assert(DR_D >= 1 && DR_D <= 128, "head sizes up to 128: the threads of a column keep it in registers");
static_assert(DR_THREADS <= 1024, "one block per head");

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

// Loads of a tile's inputs that stay where they are written (volatile): they are issued before the tile ahead is run
// and used after it; left to itself the compiler moves them down to their use and the tile then waits for memory.
__device__ __forceinline__ float ld_early(const float* p) {
  float v;
  asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ float ld_early(const bf16* p) {
  unsigned short v;
  asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return __uint_as_float((unsigned)v << 16);
}

__device__ __forceinline__ int split_index(int i) { return (i / DR_DK) * DR_LD + (i % DR_DK); }   // channel -> place

// sum over the KS neighbouring lanes that share a column (every lane of the warp takes part)
__device__ __forceinline__ float column_sum(float v) {
#pragma unroll
  for (int o = 1; o < DR_KS; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename TA, typename TW>
__global__ void __launch_bounds__(DR_THREADS) delta_rule_kernel(DeltaRuleParams p) {
  __shared__ __align__(16) float sk[DR_TT][DR_ROW], sr[DR_TT][DR_ROW], sw[DR_TT][DR_ROW], sb[DR_TT][DR_ROW],
      su[DR_TT][DR_ROW], sg[DR_TT][DR_D], sv[DR_TT][DR_D], so[DR_TT][DR_D];
  pdl_trigger();
  pdl_wait();
  const int req = blockIdx.x, h = blockIdx.y;
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  constexpr int n_warps = DR_THREADS / 32;
  const int j = tid / DR_KS, part = tid - j * DR_KS;      // this thread's column and which rows of it
  const bool active = j < DR_D;
  const int row0 = part * DR_DK;       // first row of the state this thread holds
  const int base = part * DR_LD;       // where those rows' vector elements lie in shared memory
  const int q0 = p.q_start[req], q1 = p.q_start[req + 1];
  const int slot = IE_SLOT(p.slots[req]);
  const int col0 = h * DR_D;
  TA* out = (TA*)p.out;
  if (slot < 0) {
    for (int idx = tid; idx < (q1 - q0) * DR_D; idx += DR_THREADS)
      out[(size_t)(q0 + idx / DR_D) * p.out_stride + col0 + idx % DR_D] = from_f32<TA>(0.f);
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

  float S[DR_DK];
  float* st = p.state + (((size_t)slot * p.n_heads + h) * DR_D) * DR_D;
#pragma unroll
  for (int i = 0; i < DR_DK; ++i) S[i] = active ? st[(size_t)(row0 + i) * DR_D + j] : 0.f;

  // a tile's inputs in registers: element e of the tile is (token e / D, channel e % D)
  float fk[DR_PER], fr[DR_PER], fa[DR_PER], fw[DR_PER], fg[DR_PER], fv[DR_PER];
  auto fetch = [&](int t0, int nt) {
#pragma unroll
    for (int u = 0; u < DR_PER; ++u) {
      const int e = tid + u * DR_THREADS;
      const int tt = e / DR_D, i = e - tt * DR_D;
      if (tt < nt) {
        const size_t row = (size_t)(t0 + tt) * p.stride + col0 + i;
        fk[u] = ld_early(K + row);
        fr[u] = ld_early(R + row);
        fa[u] = ld_early(A + row);
        fg[u] = ld_early(G + row);
        fv[u] = ld_early(V + row);
        fw[u] = ld_early(p.w_pre + (size_t)(t0 + tt) * p.w_stride + col0 + i);
      }
    }
  };
  if (q0 < q1) fetch(q0, min(DR_TT, q1 - q0));
  // the channel of element u of this thread is the same in every tile: its three constants are read once
  float c_ab[DR_PER], c_wb[DR_PER], c_gn[DR_PER];
#pragma unroll
  for (int u = 0; u < DR_PER; ++u) {
    const int i = (tid + u * DR_THREADS) % DR_D;
    c_ab[u] = to_f32(a_bias[col0 + i]);
    c_wb[u] = to_f32(w_bias[col0 + i]);
    c_gn[u] = to_f32(gain[col0 + i]);
  }

  for (int t0 = q0; t0 < q1; t0 += DR_TT) {
    const int nt = min(DR_TT, q1 - t0);
    // (A) the tile's vectors into shared memory, then the unit key of every token
#pragma unroll
    for (int u = 0; u < DR_PER; ++u) {
      const int e = tid + u * DR_THREADS;
      const int tt = e / DR_D, i = e - tt * DR_D;
      if (tt < nt) {
        const int si = split_index(i);
        sk[tt][si] = fk[u];
        sr[tt][si] = fr[u];
        sv[tt][i] = fv[u];
        sb[tt][si] = sigmoidf_(fa[u] + c_ab[u]);
        sw[tt][si] = expf(-p.decay_rate * sigmoidf_(fw[u] + c_wb[u]));
        sg[tt][i] = c_gn[u] * sigmoidf_(fg[u]);
      }
    }
    __syncthreads();
    for (int tt = warp; tt < nt; tt += n_warps) {
      float ss = 0.f;
      for (int i = lane; i < DR_D; i += 32) {
        const float kk = sk[tt][split_index(i)];
        ss += kk * kk;
      }
      const float knorm = sqrtf(warp_sum(ss) + p.key_eps);
      for (int i = lane; i < DR_D; i += 32) {
        const int si = split_index(i);
        const float u = sk[tt][si] / knorm;
        su[tt][si] = u;
        sb[tt][si] *= u;
      }
    }
    __syncthreads();
    if (t0 + DR_TT < q1) fetch(t0 + DR_TT, min(DR_TT, q1 - t0 - DR_TT));     // lands while this tile runs
    // (B) the tile's tokens in order; this thread's rows of its column of the state
#pragma unroll 2
    for (int tt = 0; tt < nt; ++tt) {
      float uu[DR_DK], bb[DR_DK], kk[DR_DK], ww[DR_DK], rr[DR_DK];
      if constexpr (DR_VEC) {       // 16 bytes a load: a fifth of the loads of the scalar form
#pragma unroll
        for (int i = 0; i < DR_DK; i += 4) {
          *reinterpret_cast<float4*>(&uu[i]) = *reinterpret_cast<const float4*>(&su[tt][base + i]);
          *reinterpret_cast<float4*>(&bb[i]) = *reinterpret_cast<const float4*>(&sb[tt][base + i]);
          *reinterpret_cast<float4*>(&kk[i]) = *reinterpret_cast<const float4*>(&sk[tt][base + i]);
          *reinterpret_cast<float4*>(&ww[i]) = *reinterpret_cast<const float4*>(&sw[tt][base + i]);
          *reinterpret_cast<float4*>(&rr[i]) = *reinterpret_cast<const float4*>(&sr[tt][base + i]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < DR_DK; ++i) {
          uu[i] = su[tt][base + i]; bb[i] = sb[tt][base + i]; kk[i] = sk[tt][base + i];
          ww[i] = sw[tt][base + i]; rr[i] = sr[tt][base + i];
        }
      }
      const float vj = active ? sv[tt][j] : 0.f;
      float us[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < DR_DK; ++i) us[i & 3] = fmaf(uu[i], S[i], us[i & 3]);
      const float seen = column_sum((us[0] + us[1]) + (us[2] + us[3]));
      // one pass per operation, so that neighbouring instructions do not wait for one another
      float add[DR_DK];
#pragma unroll
      for (int i = 0; i < DR_DK; ++i) add[i] = kk[i] * vj;
#pragma unroll
      for (int i = 0; i < DR_DK; ++i) add[i] = fmaf(-bb[i], seen, add[i]);
#pragma unroll
      for (int i = 0; i < DR_DK; ++i) S[i] = fmaf(ww[i], S[i], add[i]);
      float oo[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < DR_DK; ++i) oo[i & 3] = fmaf(S[i], rr[i], oo[i & 3]);
      const float o = column_sum((oo[0] + oo[1]) + (oo[2] + oo[3]));
      if (active && part == 0) so[tt][j] = o;
    }
    __syncthreads();
    // (C) norm over the head, gain, gate; a warp per token
    for (int tt = warp; tt < nt; tt += n_warps) {
      float ss = 0.f;
      for (int i = lane; i < DR_D; i += 32) ss += so[tt][i] * so[tt][i];
      const float rms = sqrtf(warp_sum(ss) / (float)DR_D + p.norm_eps);
      for (int i = lane; i < DR_D; i += 32)
        out[(size_t)(t0 + tt) * p.out_stride + col0 + i] = from_f32<TA>(so[tt][i] / rms * sg[tt][i]);
    }
    __syncthreads();
  }
  if (p.write_state && active) {
#pragma unroll
    for (int i = 0; i < DR_DK; ++i) st[(size_t)(row0 + i) * DR_D + j] = S[i];
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
