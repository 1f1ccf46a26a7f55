// Recurrent mixers with a matrix of state per head: a decaying outer-product memory ("lightning") and the gated
// delta rule.  Per head, with S [key channels][value channels] in float, carried from token to token:
//
//   lightning    S <- d S + k v^T;                               o = S^T q      d: one constant per head
//   delta rule   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q   g, beta: one number per token and head
//
// The state of a sequence lives in its slot of the cache's state region ([slots][heads][dk][dv] floats, zero when
// the slot is handed out): a step reads it, runs its tokens in order and writes it back, so a prompt in one step,
// in pieces or token by token performs the same float operations in the same order.  Query/key head of value head
// h: h / (heads / qk_heads).  Everything here is float on both paths.
//
//   hb_silu_columns     in place: x <- silu(x) on a range of columns of float rows
//   hb_delta_prepare    q, k -> unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times qscale;
//                       beta = sigmoid(b);  g = exp(-exp(A_log) * softplus(a + dt_bias))
//   hb_linear_scan      the recurrence
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
// state is held by R neighbouring lanes of one warp, RPT consecutive rows each in registers, so the two sums over
// the key channels (S^T k and S^T q) end with shuffles inside the warp and no barrier stands between two tokens.
// R and RPT follow from the head's key size alone, so that a prompt and its continuation token by token add in
// the same order.  q, k, v (and g, beta) of LS_CHUNK tokens at a time are copied into shared memory asynchronously,
// the next chunk while this one is worked on.
#define LS_THREADS 128
#define LS_CHUNK 16
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
    const int r = rg * RPT + i;
    s[i] = (r < a.dk && col < a.dv) ? S[(size_t)r * a.dv + col] : 0.0f;
  }
  for (int i = tid; i < 2 * stage_floats; i += LS_THREADS) sh[i] = 0.0f;      // rows past dk stay zero from here on
  __syncthreads();
  const bool wide = a.dk % 4 == 0 && a.ldq % 4 == 0 && a.ldk % 4 == 0 && (((uintptr_t)a.q | (uintptr_t)a.k) & 15) == 0;
  const float d = DELTA ? 0.0f : a.decay[h];

  auto stage = [&](int buf, int c0) {
    float* qs = sh + buf * stage_floats;
    float* ks = qs + LS_CHUNK * DKP;
    float* vs = ks + LS_CHUNK * DKP;
    float* gs = vs + LS_CHUNK * cols;
    const int n = t1 - c0 < LS_CHUNK ? t1 - c0 : LS_CHUNK;
    if (wide) {
      const int per = a.dk >> 2;
      for (int i = tid; i < n * per; i += LS_THREADS) {
        const int tt = i / per, r = (i - tt * per) * 4;
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
      const int tt = i / cols, c = blockIdx.z * cols + (i % cols);
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
    for (int tt = 0; tt < n; ++tt) {
      const float v = vs[tt * cols + cl];
      const float4* k4 = reinterpret_cast<const float4*>(ks + tt * DKP + rg * RPT);
      const float4* q4 = reinterpret_cast<const float4*>(qs + tt * DKP + rg * RPT);
      float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
      if (DELTA) {
        const float g = gs[2 * tt], beta = gs[2 * tt + 1];
        float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
#pragma unroll
        for (int i = 0; i < RPT / 4; ++i) {
          const float4 k = k4[i];
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
          const float4 k = k4[i], q = q4[i];
          s[4 * i] = fmaf(k.x, u, s[4 * i]);             o0 = fmaf(s[4 * i], q.x, o0);
          s[4 * i + 1] = fmaf(k.y, u, s[4 * i + 1]);     o1 = fmaf(s[4 * i + 1], q.y, o1);
          s[4 * i + 2] = fmaf(k.z, u, s[4 * i + 2]);     o2 = fmaf(s[4 * i + 2], q.z, o2);
          s[4 * i + 3] = fmaf(k.w, u, s[4 * i + 3]);     o3 = fmaf(s[4 * i + 3], q.w, o3);
        }
      } else {
#pragma unroll
        for (int i = 0; i < RPT / 4; ++i) {
          const float4 k = k4[i], q = q4[i];
          s[4 * i] = fmaf(d, s[4 * i], k.x * v);             o0 = fmaf(s[4 * i], q.x, o0);
          s[4 * i + 1] = fmaf(d, s[4 * i + 1], k.y * v);     o1 = fmaf(s[4 * i + 1], q.y, o1);
          s[4 * i + 2] = fmaf(d, s[4 * i + 2], k.z * v);     o2 = fmaf(s[4 * i + 2], q.z, o2);
          s[4 * i + 3] = fmaf(d, s[4 * i + 3], k.w * v);     o3 = fmaf(s[4 * i + 3], q.w, o3);
        }
      }
      float o = (o0 + o1) + (o2 + o3);
      for (int w = R >> 1; w > 0; w >>= 1) o += __shfl_xor_sync(0xffffffffu, o, w);
      if (rg == 0 && col < a.dv) a.out[(size_t)(c0 + tt) * a.ldo + h * a.dv + col] = o;
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = rg * RPT + i;
    if (r < a.dk && col < a.dv) S[(size_t)r * a.dv + col] = s[i];
  }
}

extern "C" int hb_linear_scan(int delta, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                              const float* gates, const float* decay, float* state, const int* seq_slot, const int* seq_start,
                              float* out, int ldo, int n_seqs, int heads, int qk_heads, int dk, int dv, void* stream) {
  HB_REQUIRE(n_seqs > 0 && heads > 0 && qk_heads > 0 && dk > 0 && dv > 0, "linear_scan: sizes must be positive");
  HB_REQUIRE(heads % qk_heads == 0, "linear_scan: %d heads are not a multiple of %d query/key heads", heads, qk_heads);
  HB_REQUIRE(dk <= 2048, "linear_scan: %d key channels per head exceed the supported maximum 2048", dk);
  HB_REQUIRE(delta ? gates != nullptr : decay != nullptr, "linear_scan: the delta rule needs its gates, the decaying form its decays");
  // lanes per column: about 16 rows per lane; the choice depends on the key size only
  int R = 1;
  while (R < 32 && R * 16 < dk) R <<= 1;
  int rpt = ceil_div(ceil_div(dk, R), 4) * 4;
  rpt = rpt <= 4 ? 4 : rpt <= 8 ? 8 : rpt <= 16 ? 16 : rpt <= 32 ? 32 : 64;
  const int cols = LS_THREADS / R;
  HB_REQUIRE(heads <= 65535 && ceil_div(dv, cols) <= 65535, "linear_scan: too many heads or value channels");
  ScanArgs a{q, ldq, k, ldk, v, ldv, gates, decay, state, seq_slot, seq_start, out, ldo, heads, qk_heads, dk, dv, R};
  dim3 grid(n_seqs, heads, ceil_div(dv, cols));
  const size_t smem = (size_t)2 * LS_CHUNK * (2 * R * rpt + cols + 2) * sizeof(float);
  cudaStream_t s = (cudaStream_t)stream;
#define LS_GO(RPT)                                                                                                              \
  do {                                                                                                                          \
    if (delta) {                                                                                                                \
      if (smem > 48 * 1024) cudaFuncSetAttribute(linear_scan_kernel<RPT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      hb_launch(linear_scan_kernel<RPT, true>, grid, dim3(LS_THREADS), smem, s, a);                                             \
    } else {                                                                                                                    \
      if (smem > 48 * 1024) cudaFuncSetAttribute(linear_scan_kernel<RPT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      hb_launch(linear_scan_kernel<RPT, false>, grid, dim3(LS_THREADS), smem, s, a);                                            \
    }                                                                                                                           \
  } while (0)
  if (rpt == 4) LS_GO(4); else if (rpt == 8) LS_GO(8); else if (rpt == 16) LS_GO(16); else if (rpt == 32) LS_GO(32); else LS_GO(64);
#undef LS_GO
  HB_CHECK_LAUNCH("linear_scan");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// y[t, u, :] = o / sqrt(mean(o^2) + eps) * w * act(gate): a unit u is one head (w [n] shared by the heads) or the whole
// row of all heads (w [units * n] ... one unit).  act: 0 silu, 1 sigmoid.  One CTA per (token, unit).
template <typename T>
__global__ void __launch_bounds__(256)
gated_rmsnorm_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ w, float eps, const float* __restrict__ gate,
                     int ldg, T* __restrict__ y, int ldy, int units, int n, int act) {
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
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float gv = g[i];
    const float sg = 1.0f / (1.0f + expf(-gv));
    yr[i] = from_f32<T>(((orow[i] * inv) * w[i]) * (act == 0 ? gv * sg : sg));
  }
}

extern "C" int hb_gated_rmsnorm(int dtype, const float* o, int ldo, const float* w, float eps, const float* gate, int ldg,
                                void* y, int ldy, int n_tokens, int units, int n, int act, void* stream) {
  HB_REQUIRE(n_tokens > 0 && units > 0 && n > 0, "gated_rmsnorm: sizes must be positive");
  HB_REQUIRE(act == 0 || act == 1, "gated_rmsnorm: the gate's activation is 0 (silu) or 1 (sigmoid)");
  const long long blocks = (long long)n_tokens * units;
  HB_REQUIRE(blocks < 2147483647LL, "gated_rmsnorm: too many (token, unit) pairs");
  const int threads = n >= 1024 ? 256 : n >= 128 ? 128 : (n >= 64 ? 64 : 32);
  if (dtype == HB_F32)
    hb_launch(gated_rmsnorm_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, (cudaStream_t)stream, o, ldo, w, eps, gate,
              ldg, (float*)y, ldy, units, n, act);
  else
    hb_launch(gated_rmsnorm_kernel<bf16>, dim3((unsigned)blocks), dim3(threads), 0, (cudaStream_t)stream, o, ldo, w, eps, gate,
              ldg, (bf16*)y, ldy, units, n, act);
  HB_CHECK_LAUNCH("gated_rmsnorm");
  return 0;
}
