// Recurrent mixers with a matrix of state per head: a decaying outer-product memory ("lightning") and the gated
// delta rule.  Per head, with S [key channels][value channels] in float, carried from token to token:
//
//   lightning    S <- d S + k v^T;                               o = S^T q      d: one constant per head
//   delta rule   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q   g, beta: one number per token and head
//
// The state of a sequence lives in its slot of the cache's state region ([slots][heads][dk][dv] floats, zero when
// the slot is handed out): a step reads it, runs its tokens in order and writes it back, so a prompt in one step,
// in pieces or token by token computes the same recurrence; the order in which a sum over the key channels is
// taken follows the launch (lanes per column, tokens one by one or sixteen at a time), so two cuttings agree to
// float rounding, not to the bit.  Query/key head of value head h: h / (heads / qk_heads).  Everything here is
// float on both paths.
//
//   hb_silu_columns     in place: x <- silu(x) on a range of columns of float rows
//   hb_delta_prepare    q, k -> unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times qscale;
//                       beta = sigmoid(b);  g = exp(-exp(A_log) * softplus(a + dt_bias))
//   hb_linear_scan      the recurrence: token by token (decode, short steps, several sequences), or for one long
//                       prompt alone the delta rule sixteen tokens at a time
//   hb_gated_rmsnorm    y = o / rms(o) * w * gate-activation(g), the norm per head (w [dv]) or over all heads (w [H dv])
#include "api.h"
#include "common.cuh"

__global__ void silu_columns_kernel(float* __restrict__ x, int ld, int col0, int cols, int rows) {
  pdl_wait();
  pdl_launch();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)rows * cols) return;
  float* p = x + (size_t)(i / cols) * ld + col0 + (int)(i % cols);
  const float v = *p;
  *p = v / (1.0f + expf(-v));
}

extern "C" int hb_silu_columns(float* x, int ld, int col0, int cols, int rows, void* stream) {
  HB_REQUIRE(rows > 0 && cols > 0, "silu_columns: sizes must be positive");
  const long long blocks = ceil_div_ll((long long)rows * cols, 256);
  HB_REQUIRE(blocks < 2147483647LL, "silu_columns: too many elements");
  hb_launch(silu_columns_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, x, ld, col0, cols, rows);
  HB_CHECK_LAUNCH("silu_columns");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// One warp per (token, q/k head) normalises q and k in place; the first warps of a token also turn the token's
// per-head numbers into beta and g.  grid: (tokens), block: 32 * warps.
__global__ void delta_prepare_kernel(float* __restrict__ qk, int ld, int q_off, int k_off, int G, int dk, float qscale,
                                     const float* __restrict__ ab, int ldab, int b_off, int a_off, const float* __restrict__ a_log,
                                     const float* __restrict__ dt_bias, float* __restrict__ gates, int H) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  for (int u = warp; u < 2 * G; u += nwarp) {
    const bool is_q = u < G;
    float* v = qk + (size_t)t * ld + (is_q ? q_off + u * dk : k_off + (u - G) * dk);
    float s = 0.0f;
    for (int i = lane; i < dk; i += 32) s = fmaf(v[i], v[i], s);
    s = warp_sum(s);
    const float f = (is_q ? qscale : 1.0f) / sqrtf(s + 1e-6f);
    for (int i = lane; i < dk; i += 32) v[i] *= f;
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float bz = ab[(size_t)t * ldab + b_off + h];
    const float az = ab[(size_t)t * ldab + a_off + h] + dt_bias[h];
    const float sp = fmaxf(az, 0.0f) + log1pf(expf(-fabsf(az)));      // softplus
    gates[(size_t)t * 2 * H + h] = expf(-expf(a_log[h]) * sp);          // g
    gates[(size_t)t * 2 * H + H + h] = 1.0f / (1.0f + expf(-bz));       // beta
  }
}

extern "C" int hb_delta_prepare(float* qk, int ld, int q_off, int k_off, int qk_heads, int dk, float qscale, const float* ab,
                                int ldab, int b_off, int a_off, const float* a_log, const float* dt_bias, float* gates,
                                int heads, int n_tokens, void* stream) {
  HB_REQUIRE(n_tokens > 0 && qk_heads > 0 && dk > 0 && heads > 0, "delta_prepare: sizes must be positive");
  hb_launch(delta_prepare_kernel, dim3(n_tokens), dim3(128), 0, (cudaStream_t)stream, qk, ld, q_off, k_off, qk_heads, dk, qscale,
            ab, ldab, b_off, a_off, a_log, dt_bias, gates, heads);
  HB_CHECK_LAUNCH("delta_prepare");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// The recurrence.  A CTA of four warps owns 128 / R value channels of one head of one sequence; a column of the
// state is held by R neighbouring lanes of one warp, RPT rows each in registers (lane g holds rows 4 (i R + g) .. + 3,
// i = 0 .. RPT / 4 - 1, so that the R lanes read neighbouring 16-byte pieces of a key and no two meet in a bank), so the two sums over
// the key channels (S^T k and S^T q) end with shuffles inside the warp and no barrier stands between two tokens.
// R and RPT follow from the head's key size and, for one long prompt alone, the grid (see the launcher).  q, k, v
// (and g, beta) of LS_CHUNK tokens at a time are copied into shared memory asynchronously, the next chunk while
// this one is worked on.
#define LS_THREADS 128
#define LS_CHUNK 16
#define LS_RED_PAD 8
__device__ __forceinline__ void ls_copy4(float* smem, const float* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void ls_copy16(float* smem, const float* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem));
}

struct ScanArgs {
  const float* q; int ldq;      // q[t * ldq + head * dk + i], head among the q/k heads
  const float* k; int ldk;
  const float* v; int ldv;      // v[t * ldv + h * dv + c]
  const float* gates;           // delta rule: [tokens][2 H]: g, then beta;  lightning: null
  const float* decay;           // lightning: [H]
  float* state;
  const int* seq_slot;
  const int* seq_start;
  float* out; int ldo;
  int H, G, dk, dv, R;
};

template <int RPT, bool DELTA>
__global__ void __launch_bounds__(LS_THREADS) linear_scan_kernel(ScanArgs a) {
  extern __shared__ __align__(16) float sh[];
  const int R = a.R, DKP = R * RPT, cols = LS_THREADS / R;
  const int stage_floats = LS_CHUNK * (2 * DKP + cols + 2);
  const int red_ld = LS_THREADS + LS_RED_PAD;
  float* red = sh + 2 * stage_floats;                             // [LS_CHUNK][cols][R]: the lanes' parts of a read-out
  pdl_wait();
  pdl_launch();
  const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int rg = lane % R;                                        // which rows of the column
  const int cl = warp * (32 / R) + lane / R;                      // column within the CTA
  const int col = blockIdx.z * cols + cl;
  const int qh = h / (a.H / a.G);
  const int t0 = a.seq_start[b], t1 = a.seq_start[b + 1];
  float* S = a.state + (((size_t)a.seq_slot[b] * a.H + h) * a.dk) * (size_t)a.dv;
  float s[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = 4 * ((i >> 2) * R + rg) + (i & 3);
    s[i] = (r < a.dk && col < a.dv) ? S[(size_t)r * a.dv + col] : 0.0f;
  }
  for (int i = tid; i < 2 * stage_floats; i += LS_THREADS) sh[i] = 0.0f;      // rows past dk stay zero from here on
  __syncthreads();
  const bool wide = a.dk % 4 == 0 && a.ldq % 4 == 0 && a.ldk % 4 == 0 && (((uintptr_t)a.q | (uintptr_t)a.k) & 15) == 0;
  const float d = DELTA ? 0.0f : a.decay[h];
  int st_lanes = 1;                                               // threads that copy one token's row of q and k
  while (st_lanes < LS_THREADS && st_lanes * 4 < a.dk) st_lanes <<= 1;
  const int st_row = tid / st_lanes, st_r = (tid % st_lanes) * 4;
  const int cshift = 31 - __clz(cols);                            // cols is a power of two

  auto stage = [&](int buf, int c0) {
    float* qs = sh + buf * stage_floats;
    float* ks = qs + LS_CHUNK * DKP;
    float* vs = ks + LS_CHUNK * DKP;
    float* gs = vs + LS_CHUNK * cols;
    const int n = t1 - c0 < LS_CHUNK ? t1 - c0 : LS_CHUNK;
    if (wide) {      // a power of two of threads per token's row, so no division stands in the loop
      for (int tt = st_row; tt < n; tt += LS_THREADS / st_lanes)
        for (int r = st_r; r < a.dk; r += st_lanes * 4) {
          ls_copy16(qs + tt * DKP + r, a.q + (size_t)(c0 + tt) * a.ldq + qh * a.dk + r);
          ls_copy16(ks + tt * DKP + r, a.k + (size_t)(c0 + tt) * a.ldk + qh * a.dk + r);
        }
    } else {
      for (int i = tid; i < n * a.dk; i += LS_THREADS) {
        const int tt = i / a.dk, r = i - tt * a.dk;
        ls_copy4(qs + tt * DKP + r, a.q + (size_t)(c0 + tt) * a.ldq + qh * a.dk + r);
        ls_copy4(ks + tt * DKP + r, a.k + (size_t)(c0 + tt) * a.ldk + qh * a.dk + r);
      }
    }
    for (int i = tid; i < n * cols; i += LS_THREADS) {
      const int tt = i >> cshift, c = blockIdx.z * cols + (i & (cols - 1));
      if (c < a.dv) ls_copy4(vs + i, a.v + (size_t)(c0 + tt) * a.ldv + h * a.dv + c);
    }
    if (DELTA)
      for (int i = tid; i < 2 * n; i += LS_THREADS) {
        const int tt = i >> 1, which = i & 1;
        ls_copy4(gs + i, a.gates + (size_t)(c0 + tt) * 2 * a.H + which * a.H + h);
      }
    asm volatile("cp.async.commit_group;");
  };

  if (t0 < t1) stage(0, t0);
  int buf = 0;
  for (int c0 = t0; c0 < t1; c0 += LS_CHUNK, buf ^= 1) {
    const int n = t1 - c0 < LS_CHUNK ? t1 - c0 : LS_CHUNK;
    if (c0 + LS_CHUNK < t1) {
      stage(buf ^ 1, c0 + LS_CHUNK);
      asm volatile("cp.async.wait_group 1;");
    } else {
      asm volatile("cp.async.wait_group 0;");
    }
    __syncthreads();
    const float* qs = sh + buf * stage_floats;
    const float* ks = qs + LS_CHUNK * DKP;
    const float* vs = ks + LS_CHUNK * DKP;
    const float* gs = vs + LS_CHUNK * cols;
    if (DELTA) {
      for (int tt = 0; tt < n; ++tt) {
        const float v = vs[tt * cols + cl];
        const float4* k4 = reinterpret_cast<const float4*>(ks + tt * DKP) + rg;
        const float4* q4 = reinterpret_cast<const float4*>(qs + tt * DKP) + rg;
        float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
        const float g = gs[2 * tt], beta = gs[2 * tt + 1];
        float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
#pragma unroll
        for (int i = 0; i < RPT / 4; ++i) {
          const float4 k = k4[i * R];
          s[4 * i] *= g;         d0 = fmaf(s[4 * i], k.x, d0);
          s[4 * i + 1] *= g;     d1 = fmaf(s[4 * i + 1], k.y, d1);
          s[4 * i + 2] *= g;     d2 = fmaf(s[4 * i + 2], k.z, d2);
          s[4 * i + 3] *= g;     d3 = fmaf(s[4 * i + 3], k.w, d3);
        }
        float dot = (d0 + d1) + (d2 + d3);
        for (int o = R >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const float u = beta * (v - dot);
#pragma unroll
        for (int i = 0; i < RPT / 4; ++i) {
          const float4 k = k4[i * R], q = q4[i * R];
          s[4 * i] = fmaf(k.x, u, s[4 * i]);             o0 = fmaf(s[4 * i], q.x, o0);
          s[4 * i + 1] = fmaf(k.y, u, s[4 * i + 1]);     o1 = fmaf(s[4 * i + 1], q.y, o1);
          s[4 * i + 2] = fmaf(k.z, u, s[4 * i + 2]);     o2 = fmaf(s[4 * i + 2], q.z, o2);
          s[4 * i + 3] = fmaf(k.w, u, s[4 * i + 3]);     o3 = fmaf(s[4 * i + 3], q.w, o3);
        }
        float o = (o0 + o1) + (o2 + o3);
        for (int w = R >> 1; w > 0; w >>= 1) o += __shfl_xor_sync(0xffffffffu, o, w);
        if (rg == 0 && col < a.dv) a.out[(size_t)(c0 + tt) * a.ldo + h * a.dv + col] = o;
      }
    } else {
      // Nothing of a token's read-out goes back into the state, so the lanes leave their parts of it in shared memory
      // and the chunk's sums are taken afterwards; between two tokens stands one multiply-add per state entry, and
      // the loop is unrolled so that the loads of several tokens are under way at once.
#pragma unroll 4
      for (int tt = 0; tt < n; ++tt) {
        const float v = vs[tt * cols + cl];
        const float4* k4 = reinterpret_cast<const float4*>(ks + tt * DKP) + rg;
        const float4* q4 = reinterpret_cast<const float4*>(qs + tt * DKP) + rg;
        float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
#pragma unroll
        for (int i = 0; i < RPT / 4; ++i) {
          const float4 k = k4[i * R], q = q4[i * R];
          s[4 * i] = fmaf(d, s[4 * i], k.x * v);             o0 = fmaf(s[4 * i], q.x, o0);
          s[4 * i + 1] = fmaf(d, s[4 * i + 1], k.y * v);     o1 = fmaf(s[4 * i + 1], q.y, o1);
          s[4 * i + 2] = fmaf(d, s[4 * i + 2], k.z * v);     o2 = fmaf(s[4 * i + 2], q.z, o2);
          s[4 * i + 3] = fmaf(d, s[4 * i + 3], k.w * v);     o3 = fmaf(s[4 * i + 3], q.w, o3);
        }
        red[tt * red_ld + cl * R + rg] = (o0 + o1) + (o2 + o3);
      }
      __syncthreads();
      for (int i = tid; i < n * cols; i += LS_THREADS) {
        const int tt = i >> cshift, c = i & (cols - 1), cc = blockIdx.z * cols + c;
        if (cc < a.dv) {
          float o = red[tt * red_ld + c * R];
          for (int g = 1; g < R; ++g) o += red[tt * red_ld + c * R + g];
          a.out[(size_t)(c0 + tt) * a.ldo + h * a.dv + cc] = o;
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = 4 * ((i >> 2) * R + rg) + (i & 3);
    if (r < a.dk && col < a.dv) S[(size_t)r * a.dv + col] = s[i];
  }
}

// ---------------------------------------------------------------------------------------------
// The same recurrence for steps that bring many tokens, LS_CHUNK at a time without a token-by-token chain over the
// state.  With S0 the state before a chunk, W[t][s] = g_(s+1) ... g_t (1 for s = t) and G[t] = g_0 ... g_t:
//
//   S_t = G[t] S0 + sum_(s<=t) W[t][s] k_s u_s^T
//   u_t = beta_t (v_t - G[t] S0^T k_t - sum_(s<t) W[t][s] (k_s . k_t) u_s)          (lightning: u_t = v_t)
//   o_t = G[t] S0^T q_t + sum_(s<=t) W[t][s] (k_s . q_t) u_s
//
// so the two products with S0 and the state's update are sums over all tokens of the chunk at once, and what is still
// taken token by token is one number per value channel (u_t, from the u_s before it).  The products of decays are
// running products (no logarithms), so a decay of zero wipes what came before it and nothing else.  The layout of
// the state is the token-by-token kernel's: a column in R neighbouring lanes, RPT rows each.  The CTA first fills the
// two small matrices M[t][s] = W (k_s . k_t) and N[t][s] = W (k_s . q_t) (one entry a thread: the upper triangle's
// threads take the mirrored entry of the lower half), while every thread multiplies its rows of S0 with the chunk's
// keys and queries.
template <bool V> struct ls_const { static constexpr bool value = V; };
#define LS_CHUNKED_FROM 8
#define LS_KPAD 4      // a token's row of keys in shared memory is this much longer: rows of neighbouring tokens in other banks
static_assert(LS_CHUNK == 16 && LS_THREADS == 128, "the chunked scan maps one entry of a 16 x 16 triangle to each of 128 threads");

template <int RPT, bool DELTA>
__global__ void __launch_bounds__(LS_THREADS) linear_scan_chunked_kernel(ScanArgs a) {
  extern __shared__ __align__(16) float sh[];
  constexpr int C = LS_CHUNK;
  const int R = a.R, DKP = R * RPT, KS = DKP + LS_KPAD, cols = LS_THREADS / R;
  const int stage_floats = C * (2 * KS + cols + 2);
  float* Mm = sh + 2 * stage_floats;       // [C][C]
  float* Nn = Mm + C * C;                  // [C][C]
  float* Gt = Nn + C * C;                  // [C]: decay from before the chunk through token t
  float* Et = Gt + C;                      // [C]: decay from after token t to the chunk's end
  pdl_wait();
  pdl_launch();
  const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int rg = lane % R;
  const int cl = warp * (32 / R) + lane / R;
  const int col = blockIdx.z * cols + cl;
  const int qh = h / (a.H / a.G);
  const int t0 = a.seq_start[b], t1 = a.seq_start[b + 1];
  float* S = a.state + (((size_t)a.seq_slot[b] * a.H + h) * a.dk) * (size_t)a.dv;
  float s[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = 4 * ((i >> 2) * R + rg) + (i & 3);
    s[i] = (r < a.dk && col < a.dv) ? S[(size_t)r * a.dv + col] : 0.0f;
  }
  for (int i = tid; i < 2 * stage_floats + 2 * C * C + 2 * C; i += LS_THREADS) sh[i] = 0.0f;
  __syncthreads();
  const bool wide = a.dk % 4 == 0 && a.ldq % 4 == 0 && a.ldk % 4 == 0 && (((uintptr_t)a.q | (uintptr_t)a.k) & 15) == 0;
  const float d = DELTA ? 0.0f : a.decay[h];
  int st_lanes = 1;                                               // threads that copy one token's row of q and k
  while (st_lanes < LS_THREADS && st_lanes * 4 < a.dk) st_lanes <<= 1;
  const int st_row = tid / st_lanes, st_r = (tid % st_lanes) * 4;
  const int cshift = 31 - __clz(cols);                            // cols is a power of two

  auto stage = [&](int buf, int c0) {
    float* qs = sh + buf * stage_floats;
    float* ks = qs + C * KS;
    float* vs = ks + C * KS;
    float* gs = vs + C * cols;
    const int n = t1 - c0 < C ? t1 - c0 : C;
    if (wide) {      // a power of two of threads per token's row, so no division stands in the loop
      for (int tt = st_row; tt < n; tt += LS_THREADS / st_lanes)
        for (int r = st_r; r < a.dk; r += st_lanes * 4) {
          ls_copy16(qs + tt * KS + r, a.q + (size_t)(c0 + tt) * a.ldq + qh * a.dk + r);
          ls_copy16(ks + tt * KS + r, a.k + (size_t)(c0 + tt) * a.ldk + qh * a.dk + r);
        }
    } else {
      for (int i = tid; i < n * a.dk; i += LS_THREADS) {
        const int tt = i / a.dk, r = i - tt * a.dk;
        ls_copy4(qs + tt * KS + r, a.q + (size_t)(c0 + tt) * a.ldq + qh * a.dk + r);
        ls_copy4(ks + tt * KS + r, a.k + (size_t)(c0 + tt) * a.ldk + qh * a.dk + r);
      }
    }
    for (int i = tid; i < n * cols; i += LS_THREADS) {
      const int tt = i >> cshift, c = blockIdx.z * cols + (i & (cols - 1));
      if (c < a.dv) ls_copy4(vs + i, a.v + (size_t)(c0 + tt) * a.ldv + h * a.dv + c);
    }
    if (DELTA)
      for (int i = tid; i < 2 * n; i += LS_THREADS) {
        const int tt = i >> 1, which = i & 1;
        ls_copy4(gs + i, a.gates + (size_t)(c0 + tt) * 2 * a.H + which * a.H + h);
      }
    asm volatile("cp.async.commit_group;");
  };

  if (t0 < t1) stage(0, t0);
  int buf = 0;
  for (int c0 = t0; c0 < t1; c0 += C, buf ^= 1) {
    const int n = t1 - c0 < C ? t1 - c0 : C;
    if (c0 + C < t1) {
      stage(buf ^ 1, c0 + C);
      asm volatile("cp.async.wait_group 1;");
    } else {
      asm volatile("cp.async.wait_group 0;");
    }
    __syncthreads();
    const float* qs = sh + buf * stage_floats;
    const float* ks = qs + C * KS;
    const float* vs = ks + C * KS;
    const float* gs = vs + C * cols;

    // A full chunk runs the same statements without the tests on t, as one straight run of instructions in which the
    // loads of all tokens go ahead of the sums and the sums of different tokens interleave.
    auto work = [&](auto full_chunk) {
      constexpr bool FULL = decltype(full_chunk)::value;
      // -- the chunk's two triangles: thread -> entry (t, s), s <= t ------------------------------
      auto entry = [&](int t, int sx) {
        if (!FULL && t >= n) return;
        const float4* kt = reinterpret_cast<const float4*>(ks + t * KS);
        const float4* qt = reinterpret_cast<const float4*>(qs + t * KS);
        const float4* kk = reinterpret_cast<const float4*>(ks + sx * KS);
        const bool below = DELTA && sx < t;
        float m0 = 0.0f, m1 = 0.0f, n0 = 0.0f, n1 = 0.0f;
#pragma unroll 4
        for (int i = 0; i < DKP / 4; ++i) {
          const float4 x = kk[i], y = qt[i];
          n0 = fmaf(x.x, y.x, n0); n1 = fmaf(x.y, y.y, n1); n0 = fmaf(x.z, y.z, n0); n1 = fmaf(x.w, y.w, n1);
          if (below) {
            const float4 z = kt[i];
            m0 = fmaf(x.x, z.x, m0); m1 = fmaf(x.y, z.y, m1); m0 = fmaf(x.z, z.z, m0); m1 = fmaf(x.w, z.w, m1);
          }
        }
        float w = 1.0f;                                                 // g_(s+1) ... g_t
        for (int r = sx + 1; r <= t; ++r) w *= DELTA ? gs[2 * r] : d;
        Nn[t * C + sx] = w * (n0 + n1);
        if (below) Mm[t * C + sx] = w * (m0 + m1);
        if (sx == 0) Gt[t] = w * (DELTA ? gs[0] : d);
        if (t == n - 1) Et[sx] = w;
      };
      {
        int t = tid >> 4, sx = tid & 15;
        if (sx > t) { t = C - 1 - t; sx = C - 1 - sx; }
        entry(t, sx);
        if (tid < C / 2) entry(C / 2 + tid, C / 2 + tid);
      }

      // -- S0^T k_t and S0^T q_t for every token of the chunk -------------------------------------
      float pk[C], pq[C];
#pragma unroll
      for (int t = 0; t < C; ++t) {
        pk[t] = 0.0f; pq[t] = 0.0f;
        if (FULL || t < n) {
          const float4* k4 = reinterpret_cast<const float4*>(ks + t * KS) + rg;
          const float4* q4 = reinterpret_cast<const float4*>(qs + t * KS) + rg;
          float p0 = 0.0f, p1 = 0.0f, o0 = 0.0f, o1 = 0.0f;
#pragma unroll
          for (int i = 0; i < RPT / 4; ++i) {
            const float4 q = q4[i * R];
            o0 = fmaf(s[4 * i], q.x, o0); o1 = fmaf(s[4 * i + 1], q.y, o1);
            o0 = fmaf(s[4 * i + 2], q.z, o0); o1 = fmaf(s[4 * i + 3], q.w, o1);
            if (DELTA) {
              const float4 k = k4[i * R];
              p0 = fmaf(s[4 * i], k.x, p0); p1 = fmaf(s[4 * i + 1], k.y, p1);
              p0 = fmaf(s[4 * i + 2], k.z, p0); p1 = fmaf(s[4 * i + 3], k.w, p1);
            }
          }
          pk[t] = p0 + p1; pq[t] = o0 + o1;
        }
      }
      for (int w = R >> 1; w > 0; w >>= 1) {
#pragma unroll
        for (int t = 0; t < C; ++t) {
          pq[t] += __shfl_xor_sync(0xffffffffu, pq[t], w);
          if (DELTA) pk[t] += __shfl_xor_sync(0xffffffffu, pk[t], w);
        }
      }
      __syncthreads();                      // the triangles are complete

      // -- token by token: one number per value channel --------------------------------------------
      float u[C], o[C];
#pragma unroll
      for (int t = 0; t < C; ++t) {
        u[t] = 0.0f; o[t] = 0.0f;
        if (FULL || t < n) {
          const float v = vs[t * cols + cl];
          const float G = Gt[t];
          float row[C];                                  // a row of a triangle, four entries a load
          if (DELTA) {
#pragma unroll
            for (int j = 0; 4 * j < t; ++j) {
              const float4 x = reinterpret_cast<const float4*>(Mm + t * C)[j];
              row[4 * j] = x.x; row[4 * j + 1] = x.y; row[4 * j + 2] = x.z; row[4 * j + 3] = x.w;
            }
            float acc = fmaf(-G, pk[t], v);
#pragma unroll
            for (int sx = 0; sx < t; ++sx) acc = fmaf(-row[sx], u[sx], acc);
            u[t] = gs[2 * t + 1] * acc;
          } else {
            u[t] = v;
          }
#pragma unroll
          for (int j = 0; 4 * j <= t; ++j) {
            const float4 x = reinterpret_cast<const float4*>(Nn + t * C)[j];
            row[4 * j] = x.x; row[4 * j + 1] = x.y; row[4 * j + 2] = x.z; row[4 * j + 3] = x.w;
          }
          float acc = G * pq[t];
#pragma unroll
          for (int sx = 0; sx <= t; ++sx) acc = fmaf(row[sx], u[sx], acc);
          o[t] = acc;
        }
      }

      // -- the state after the chunk -----------------------------------------------------------------
      const float Gn = Gt[n - 1];
#pragma unroll
      for (int i = 0; i < RPT; ++i) s[i] *= Gn;
#pragma unroll
      for (int t = 0; t < C; ++t) {
        if (FULL || t < n) {
          const float eu = Et[t] * u[t];
          const float4* k4 = reinterpret_cast<const float4*>(ks + t * KS) + rg;
#pragma unroll
          for (int i = 0; i < RPT / 4; ++i) {
            const float4 k = k4[i * R];
            s[4 * i] = fmaf(k.x, eu, s[4 * i]);         s[4 * i + 1] = fmaf(k.y, eu, s[4 * i + 1]);
            s[4 * i + 2] = fmaf(k.z, eu, s[4 * i + 2]); s[4 * i + 3] = fmaf(k.w, eu, s[4 * i + 3]);
          }
        }
      }
      if (rg == 0 && col < a.dv) {
#pragma unroll
        for (int t = 0; t < C; ++t)
          if (FULL || t < n) a.out[(size_t)(c0 + t) * a.ldo + h * a.dv + col] = o[t];
      }
    };
    if (n == C) work(ls_const<true>{}); else work(ls_const<false>{});
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = 4 * ((i >> 2) * R + rg) + (i & 3);
    if (r < a.dk && col < a.dv) S[(size_t)r * a.dv + col] = s[i];
  }
}

extern "C" int hb_linear_scan(int delta, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                              const float* gates, const float* decay, float* state, const int* seq_slot, const int* seq_start,
                              float* out, int ldo, int n_seqs, int max_q_len, int heads, int qk_heads, int dk, int dv,
                              void* stream) {
  HB_REQUIRE(n_seqs > 0 && heads > 0 && qk_heads > 0 && dk > 0 && dv > 0, "linear_scan: sizes must be positive");
  HB_REQUIRE(heads % qk_heads == 0, "linear_scan: %d heads are not a multiple of %d query/key heads", heads, qk_heads);
  HB_REQUIRE(dk <= 2048, "linear_scan: %d key channels per head exceed the supported maximum 2048", dk);
  HB_REQUIRE(delta ? gates != nullptr : decay != nullptr, "linear_scan: the delta rule needs its gates, the decaying form its decays");
  // lanes per column: about 16 rows per lane, 8 when that grid would leave more than half of the SMs without a CTA
  // (one long prompt alone).  The state in memory does not depend on the choice; the order of the sums does.
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int R = 1;
  while (R < 32 && R * 16 < dk) R <<= 1;
  if (R < 32 && dk >= 8 * R && 2LL * n_seqs * heads * ceil_div(dv, LS_THREADS / R) <= sms) R <<= 1;
  int rpt = ceil_div(ceil_div(dk, R), 4) * 4;
  rpt = rpt <= 4 ? 4 : rpt <= 8 ? 8 : rpt <= 16 ? 16 : rpt <= 32 ? 32 : 64;
  const int cols = LS_THREADS / R;
  HB_REQUIRE(heads <= 65535 && ceil_div(dv, cols) <= 65535, "linear_scan: too many heads or value channels");
  ScanArgs a{q, ldq, k, ldk, v, ldv, gates, decay, state, seq_slot, seq_start, out, ldo, heads, qk_heads, dk, dv, R};
  dim3 grid(n_seqs, heads, ceil_div(dv, cols));
  // The delta rule takes the chunked kernel when the step's longest sequence brings LS_CHUNKED_FROM tokens or more and
  // the grid leaves SMs with one CTA or none: there a CTA's time is the length of its chain of dependent operations,
  // which the chunked form shortens.  With several CTAs on every SM the token-by-token form issues fewer instructions.
  const bool chunked = delta && max_q_len >= LS_CHUNKED_FROM && (long long)grid.x * grid.y * grid.z < 2LL * sms;
  const size_t smem = chunked ? (size_t)(2 * LS_CHUNK * (2 * (R * rpt + LS_KPAD) + cols + 2) + 2 * LS_CHUNK * LS_CHUNK + 2 * LS_CHUNK) * sizeof(float)
                              : (size_t)(2 * LS_CHUNK * (2 * R * rpt + cols + 2) + LS_CHUNK * (LS_THREADS + LS_RED_PAD)) * sizeof(float);
  HB_REQUIRE(smem <= 200 * 1024, "linear_scan: %d key channels per head need %zu bytes of shared memory, more than a CTA has", dk, smem);
  cudaStream_t s = (cudaStream_t)stream;
#define LS_GO_ONE(KERNEL)                                                                                                       \
  do {                                                                                                                          \
    if (smem > 48 * 1024) cudaFuncSetAttribute(KERNEL, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                 \
    hb_launch(KERNEL, grid, dim3(LS_THREADS), smem, s, a);                                                                      \
  } while (0)
#define LS_GO(RPT)                                                                                                              \
  do {                                                                                                                          \
    if (chunked) {                                                                                                              \
      if (delta) LS_GO_ONE((linear_scan_chunked_kernel<RPT, true>)); else LS_GO_ONE((linear_scan_chunked_kernel<RPT, false>));  \
    } else if (delta) {                                                                                                                \
      if (smem > 48 * 1024) cudaFuncSetAttribute(linear_scan_kernel<RPT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      hb_launch(linear_scan_kernel<RPT, true>, grid, dim3(LS_THREADS), smem, s, a);                                             \
    } else {                                                                                                                    \
      if (smem > 48 * 1024) cudaFuncSetAttribute(linear_scan_kernel<RPT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      hb_launch(linear_scan_kernel<RPT, false>, grid, dim3(LS_THREADS), smem, s, a);                                            \
    }                                                                                                                           \
  } while (0)
  if (rpt == 4) LS_GO(4); else if (rpt == 8) LS_GO(8); else if (rpt == 16) LS_GO(16); else if (rpt == 32) LS_GO(32); else LS_GO(64);
#undef LS_GO
#undef LS_GO_ONE
  HB_CHECK_LAUNCH("linear_scan");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// y[t, u, :] = o / sqrt(mean(o^2) + eps) * w * act(gate): a unit u is one head (w [n] shared by the heads, or with
// w_stride = n a weight [units * n] with a part for every head) or the whole row of all heads (one unit).
// act: 0 silu, 1 sigmoid.  One CTA per (token, unit).
template <typename T>
__global__ void __launch_bounds__(256)
gated_rmsnorm_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ w, float eps, const float* __restrict__ gate,
                     int ldg, T* __restrict__ y, int ldy, int units, int n, int act, int w_stride) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x / units, u = blockIdx.x % units;
  const float* orow = o + (size_t)t * ldo + (size_t)u * n;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(orow[i], orow[i], ss);
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  const float* g = gate + (size_t)t * ldg + (size_t)u * n;
  T* yr = y + (size_t)t * ldy + (size_t)u * n;
  w += (size_t)u * w_stride;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float gv = g[i];
    const float sg = 1.0f / (1.0f + expf(-gv));
    yr[i] = from_f32<T>(((orow[i] * inv) * w[i]) * (act == 0 ? gv * sg : sg));
  }
}

extern "C" int hb_gated_rmsnorm(int dtype, const float* o, int ldo, const float* w, float eps, const float* gate, int ldg,
                                void* y, int ldy, int n_tokens, int units, int n, int act, int w_stride, void* stream) {
  HB_REQUIRE(n_tokens > 0 && units > 0 && n > 0, "gated_rmsnorm: sizes must be positive");
  HB_REQUIRE(act == 0 || act == 1, "gated_rmsnorm: the gate's activation is 0 (silu) or 1 (sigmoid)");
  HB_REQUIRE(w_stride == 0 || w_stride == n, "gated_rmsnorm: the weight is shared by the units (stride 0) or has a part for each (stride %d)", n);
  const long long blocks = (long long)n_tokens * units;
  HB_REQUIRE(blocks < 2147483647LL, "gated_rmsnorm: too many (token, unit) pairs");
  const int threads = n >= 1024 ? 256 : n >= 128 ? 128 : (n >= 64 ? 64 : 32);
  if (dtype == HB_F32)
    hb_launch(gated_rmsnorm_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, (cudaStream_t)stream, o, ldo, w, eps, gate,
              ldg, (float*)y, ldy, units, n, act, w_stride);
  else
    hb_launch(gated_rmsnorm_kernel<bf16>, dim3((unsigned)blocks), dim3(threads), 0, (cudaStream_t)stream, o, ldo, w, eps, gate,
              ldg, (bf16*)y, ldy, units, n, act, w_stride);
  HB_CHECK_LAUNCH("gated_rmsnorm");
  return 0;
}
