// The generalised delta rule: a matrix of state per head with a decay per key channel, from which the part that
// lies along the token's unit key is taken out (channel by channel at a rate a) before k v^T is added.  Per head,
// with S [key channels][value channels] in float, carried from token to token:
//
//   u_t = k_t / sqrt(sum k_t^2 + unit_eps)
//   S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T          both terms read the old state
//   o_t = S_t^T r_t
//   w_t = exp(-c * sigmoid(W2 tanh(low_t) + w0)),   a_t = sigmoid(A h_t + a0)   one of each per head and key channel
//
// The gated delta rule (S <- g S; S <- S + beta k (v - S^T k)^T) is the case w = g, a * u -> beta g k, u -> k, k -> beta k.
//
// The state of a sequence lives in its slot of the cache's state region ([slots][heads][dk][dv] floats, zero when the
// slot is handed out): a step reads it, runs its tokens in order and writes it back, so a prompt in one step, in
// pieces or token by token performs the same float operations in the same order.  Everything here is float on both
// paths; only W2 arrives in the compute type (its products are exact, the sums float).
//
//   hb_general_delta_prepare   from the projection's float rows: the five key-side vectors of every (token, head),
//                              packed as [T][H][5][dk]: r, k, w, u, a * u
//   hb_general_delta_scan      the recurrence
#include "api.h"
#include "common.cuh"

// ---------------------------------------------------------------------------------------------
// A CTA takes one head of GP_TOK tokens, a thread one key channel of it (a head wider than the block: several): the
// thread reads its row of W2 once for all of the CTA's tokens, whose low-rank rows (after tanh) lie in shared memory;
// the sums of k^2 go through the block.  Few tokens (a decode step) still spread over heads x token groups CTAs.
#define GP_TOK 8
#define GP_MAX_THREADS 256
struct GdPrepArgs {
  const float* rows; int ld;       // the projection's float rows
  int r_off, k_off, a_off, low_off;
  const void* w2;                  // [H dk][rank], compute type
  const float* w0;                 // [H dk]
  const float* a0;                 // [H dk]
  float decay_c, unit_eps;
  float* prep;                     // [T][H][5][dk]
  int n_tokens, H, dk, rank;
};

template <typename T>
__global__ void __launch_bounds__(GP_MAX_THREADS) general_delta_prepare_kernel(GdPrepArgs a) {
  extern __shared__ float lows[];   // [GP_TOK][rank]
  __shared__ float red[GP_TOK][GP_MAX_THREADS / 32];
  __shared__ float inv[GP_TOK];
  pdl_wait();
  pdl_launch();
  const int t0 = blockIdx.x * GP_TOK, h = blockIdx.y;
  const int nt = a.n_tokens - t0 < GP_TOK ? a.n_tokens - t0 : GP_TOK;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  for (int i = threadIdx.x; i < nt * a.rank; i += blockDim.x) {
    const int tt = i / a.rank, j = i - tt * a.rank;
    lows[i] = tanhf(a.rows[(size_t)(t0 + tt) * a.ld + a.low_off + j]);
  }
  // sum of k^2 per token over the head's channels
  float ss[GP_TOK];
#pragma unroll
  for (int tt = 0; tt < GP_TOK; ++tt) ss[tt] = 0.0f;
  for (int i = threadIdx.x; i < a.dk; i += blockDim.x) {
#pragma unroll
    for (int tt = 0; tt < GP_TOK; ++tt)
      if (tt < nt) {
        const float k = a.rows[(size_t)(t0 + tt) * a.ld + a.k_off + (size_t)h * a.dk + i];
        ss[tt] = fmaf(k, k, ss[tt]);
      }
  }
#pragma unroll
  for (int tt = 0; tt < GP_TOK; ++tt) {
    const float v = warp_sum(ss[tt]);
    if (lane == 0) red[tt][warp] = v;
  }
  __syncthreads();
  if (threadIdx.x < GP_TOK) {
    float v = 0.0f;
    for (int w = 0; w < nwarp; ++w) v += red[threadIdx.x][w];
    inv[threadIdx.x] = 1.0f / sqrtf(v + a.unit_eps);
  }
  __syncthreads();
  const T* w2 = (const T*)a.w2;
  for (int i = threadIdx.x; i < a.dk; i += blockDim.x) {
    const int c = h * a.dk + i;
    const T* wr = w2 + (size_t)c * a.rank;
    float z[GP_TOK];
    const float z0 = a.w0[c], a0 = a.a0[c];
#pragma unroll
    for (int tt = 0; tt < GP_TOK; ++tt) z[tt] = z0;
    for (int j = 0; j < a.rank; ++j) {
      const float w = to_f32(wr[j]);
#pragma unroll
      for (int tt = 0; tt < GP_TOK; ++tt)
        if (tt < nt) z[tt] = fmaf(lows[tt * a.rank + j], w, z[tt]);
    }
#pragma unroll
    for (int tt = 0; tt < GP_TOK; ++tt)
      if (tt < nt) {
        const float* row = a.rows + (size_t)(t0 + tt) * a.ld;
        float* out = a.prep + ((size_t)(t0 + tt) * a.H + h) * 5 * a.dk;
        const float w = expf(-a.decay_c / (1.0f + expf(-z[tt])));
        const float rate = 1.0f / (1.0f + expf(-(row[a.a_off + c] + a0)));
        const float k = row[a.k_off + c], u = k * inv[tt];
        out[i] = row[a.r_off + c];
        out[a.dk + i] = k;
        out[2 * a.dk + i] = w;
        out[3 * a.dk + i] = u;
        out[4 * a.dk + i] = rate * u;
      }
  }
}

extern "C" int hb_general_delta_prepare(int dtype, const float* rows, int ld, int r_off, int k_off, int a_off, int low_off,
                                        const void* w2, const float* w0, const float* a0, float decay_c, float unit_eps,
                                        float* prep, int n_tokens, int heads, int dk, int rank, void* stream) {
  HB_REQUIRE(n_tokens > 0 && heads > 0 && dk > 0 && rank > 0, "general_delta_prepare: sizes must be positive");
  const size_t smem = (size_t)GP_TOK * rank * sizeof(float);
  HB_REQUIRE(smem <= 40 * 1024, "general_delta_prepare: the decay's inner width %d exceeds what a block keeps in shared memory", rank);
  HB_REQUIRE(heads <= 65535, "general_delta_prepare: too many heads");
  GdPrepArgs a{rows, ld, r_off, k_off, a_off, low_off, w2, w0, a0, decay_c, unit_eps, prep, n_tokens, heads, dk, rank};
  dim3 grid(ceil_div(n_tokens, GP_TOK), heads);
  const int threads = dk >= GP_MAX_THREADS ? GP_MAX_THREADS : ceil_div(dk, 32) * 32;
  if (dtype == HB_F32)
    hb_launch(general_delta_prepare_kernel<float>, grid, dim3(threads), smem, (cudaStream_t)stream, a);
  else
    hb_launch(general_delta_prepare_kernel<bf16>, grid, dim3(threads), smem, (cudaStream_t)stream, a);
  HB_CHECK_LAUNCH("general_delta_prepare");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// The recurrence.  A CTA of four warps owns 128 / R value channels of one head of one sequence; a column of the
// state is held by R neighbouring lanes of one warp, RPT rows each in registers (lane g holds rows 4 (i R + g) .. + 3,
// i = 0 .. RPT / 4 - 1, so that the R lanes read neighbouring 16-byte pieces of a vector and no two meet in a bank).
// A token costs two sums over the key channels, the second after the first (u^T S before the update, S^T r after
// it); both end with shuffles inside the warp, so no barrier stands between two tokens.  The five key-side vectors
// and the values of GD_CHUNK tokens at a time are copied into shared memory asynchronously, the next chunk while
// this one is worked on.
#define GD_THREADS 128
#define GD_CHUNK 16
__device__ __forceinline__ void gd_copy4(float* smem, const float* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void gd_copy16(float* smem, const float* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem));
}

struct GdScanArgs {
  const float* prep;            // [T][H][5][dk]
  const float* v; int ldv;      // v[t * ldv + h * dv + c]
  float* state;
  const int* seq_slot;
  const int* seq_start;
  float* out; int ldo;
  int H, dk, dv, R;
  int chunk;                    // tokens per stage: GD_CHUNK, fewer where a head's key channels are many
};

template <int RPT>
__global__ void __launch_bounds__(GD_THREADS) general_delta_scan_kernel(GdScanArgs a) {
  extern __shared__ __align__(16) float sh[];
  __shared__ float outs[GD_CHUNK * GD_THREADS];                   // [GD_CHUNK][cols]: a chunk's read-outs
  const int R = a.R, DKP = R * RPT, cols = GD_THREADS / R;
  const int CH = a.chunk;
  const int stage_floats = CH * (5 * DKP + cols);
  pdl_wait();
  pdl_launch();
  const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int rg = lane % R;                                        // which rows of the column
  const int cl = warp * (32 / R) + lane / R;                      // column within the CTA
  const int col = blockIdx.z * cols + cl;
  const int t0 = a.seq_start[b], t1 = a.seq_start[b + 1];
  float* S = a.state + (((size_t)a.seq_slot[b] * a.H + h) * a.dk) * (size_t)a.dv;
  float s[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = 4 * ((i >> 2) * R + rg) + (i & 3);
    s[i] = (r < a.dk && col < a.dv) ? S[(size_t)r * a.dv + col] : 0.0f;
  }
  for (int i = tid; i < 2 * stage_floats; i += GD_THREADS) sh[i] = 0.0f;      // rows past dk stay zero from here on
  __syncthreads();
  const bool wide = a.dk % 4 == 0 && (((uintptr_t)a.prep) & 15) == 0;
  const int cshift = 31 - __clz(cols);                            // cols is a power of two

  auto stage = [&](int buf, int c0) {
    float* ks = sh + buf * stage_floats;                          // [GD_CHUNK][5][DKP]
    float* vs = ks + CH * 5 * DKP;                                // [chunk][cols]
    const int n = t1 - c0 < CH ? t1 - c0 : CH;
    if (wide) {
      const int per = a.dk >> 2;
      for (int i = tid; i < n * 5 * per; i += GD_THREADS) {
        const int tv = i / per, r = (i - tv * per) * 4;           // tv = token * 5 + vector
        gd_copy16(ks + tv * DKP + r, a.prep + ((size_t)(c0 + tv / 5) * a.H + h) * 5 * a.dk + (size_t)(tv % 5) * a.dk + r);
      }
    } else {
      for (int i = tid; i < n * 5 * a.dk; i += GD_THREADS) {
        const int tv = i / a.dk, r = i - tv * a.dk;
        gd_copy4(ks + tv * DKP + r, a.prep + ((size_t)(c0 + tv / 5) * a.H + h) * 5 * a.dk + (size_t)(tv % 5) * a.dk + r);
      }
    }
    for (int i = tid; i < n * cols; i += GD_THREADS) {
      const int tt = i >> cshift, c = blockIdx.z * cols + (i & (cols - 1));
      if (c < a.dv) gd_copy4(vs + i, a.v + (size_t)(c0 + tt) * a.ldv + h * a.dv + c);
    }
    asm volatile("cp.async.commit_group;");
  };

  if (t0 < t1) stage(0, t0);
  int buf = 0;
  for (int c0 = t0; c0 < t1; c0 += CH, buf ^= 1) {
    const int n = t1 - c0 < CH ? t1 - c0 : CH;
    if (c0 + CH < t1) {
      stage(buf ^ 1, c0 + CH);
      asm volatile("cp.async.wait_group 1;");
    } else {
      asm volatile("cp.async.wait_group 0;");
    }
    __syncthreads();
    const float* ks = sh + buf * stage_floats;
    const float* vs = ks + CH * 5 * DKP;
    // Only `seen` of one token stands between it and the next: the read-out's sum and its shuffles belong to no chain, so
    // the loop is unrolled for them to run beside the next token's first sum; the results leave through an array of their
    // own in shared memory (a store into global memory in the loop would keep the next tokens' loads behind it).
#pragma unroll 4
    for (int tt = 0; tt < n; ++tt) {
      const float4* r4 = reinterpret_cast<const float4*>(ks + (tt * 5 + 0) * DKP) + rg;
      const float4* k4 = reinterpret_cast<const float4*>(ks + (tt * 5 + 1) * DKP) + rg;
      const float4* w4 = reinterpret_cast<const float4*>(ks + (tt * 5 + 2) * DKP) + rg;
      const float4* u4 = reinterpret_cast<const float4*>(ks + (tt * 5 + 3) * DKP) + rg;
      const float4* p4 = reinterpret_cast<const float4*>(ks + (tt * 5 + 4) * DKP) + rg;
      const float v = vs[tt * cols + cl];
      float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
#pragma unroll
      for (int i = 0; i < RPT / 4; ++i) {
        const float4 u = u4[i * R];
        d0 = fmaf(s[4 * i], u.x, d0);
        d1 = fmaf(s[4 * i + 1], u.y, d1);
        d2 = fmaf(s[4 * i + 2], u.z, d2);
        d3 = fmaf(s[4 * i + 3], u.w, d3);
      }
      float seen = (d0 + d1) + (d2 + d3);                          // u^T S_(t-1) for this column
      for (int o = R >> 1; o > 0; o >>= 1) seen += __shfl_xor_sync(0xffffffffu, seen, o);
      float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
#pragma unroll
      for (int i = 0; i < RPT / 4; ++i) {
        const float4 w = w4[i * R], p = p4[i * R], k = k4[i * R], r = r4[i * R];
        s[4 * i] = fmaf(w.x, s[4 * i], fmaf(-p.x, seen, k.x * v));                 o0 = fmaf(s[4 * i], r.x, o0);
        s[4 * i + 1] = fmaf(w.y, s[4 * i + 1], fmaf(-p.y, seen, k.y * v));         o1 = fmaf(s[4 * i + 1], r.y, o1);
        s[4 * i + 2] = fmaf(w.z, s[4 * i + 2], fmaf(-p.z, seen, k.z * v));         o2 = fmaf(s[4 * i + 2], r.z, o2);
        s[4 * i + 3] = fmaf(w.w, s[4 * i + 3], fmaf(-p.w, seen, k.w * v));         o3 = fmaf(s[4 * i + 3], r.w, o3);
      }
      float o = (o0 + o1) + (o2 + o3);
      for (int w = R >> 1; w > 0; w >>= 1) o += __shfl_xor_sync(0xffffffffu, o, w);
      if (rg == 0) outs[tt * cols + cl] = o;
    }
    __syncthreads();
    for (int i = tid; i < n * cols; i += GD_THREADS) {
      const int tt = i >> cshift, c = blockIdx.z * cols + (i & (cols - 1));
      if (c < a.dv) a.out[(size_t)(c0 + tt) * a.ldo + h * a.dv + c] = outs[i];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = 4 * ((i >> 2) * R + rg) + (i & 3);
    if (r < a.dk && col < a.dv) S[(size_t)r * a.dv + col] = s[i];
  }
}

extern "C" int hb_general_delta_scan(const float* prep, const float* v, int ldv, float* state, const int* seq_slot,
                                     const int* seq_start, float* out, int ldo, int n_seqs, int heads, int dk, int dv,
                                     void* stream) {
  HB_REQUIRE(n_seqs > 0 && heads > 0 && dk > 0 && dv > 0, "general_delta_scan: sizes must be positive");
  HB_REQUIRE(dk <= 1024, "general_delta_scan: %d key channels per head exceed the supported maximum 1024", dk);
  // lanes per column: about 8 rows per lane; 4 when that grid would leave more than half of the SMs without a CTA.
  // The state in memory does not depend on the choice; the order of the sums over the key channels does.
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int R = 1;
  while (R < 32 && R * 8 < dk) R <<= 1;
  if (R < 32 && dk >= 8 * R && 2LL * n_seqs * heads * ceil_div(dv, GD_THREADS / R) <= sms) R <<= 1;
  int rpt = ceil_div(ceil_div(dk, R), 4) * 4;
  rpt = rpt <= 4 ? 4 : rpt <= 8 ? 8 : rpt <= 16 ? 16 : 32;
  const int cols = GD_THREADS / R;
  HB_REQUIRE(heads <= 65535 && ceil_div(dv, cols) <= 65535, "general_delta_scan: too many heads or value channels");
  int chunk = GD_CHUNK;
  while (chunk > 2 && (size_t)2 * chunk * (5 * R * rpt + cols) * sizeof(float) > 160 * 1024) chunk >>= 1;
  const size_t smem = (size_t)2 * chunk * (5 * R * rpt + cols) * sizeof(float);
  HB_REQUIRE(smem <= 192 * 1024, "general_delta_scan: %d key channels per head need %zu bytes of shared memory, more than a CTA has", dk, smem);
  GdScanArgs a{prep, v, ldv, state, seq_slot, seq_start, out, ldo, heads, dk, dv, R, chunk};
  dim3 grid(n_seqs, heads, ceil_div(dv, cols));
  cudaStream_t s = (cudaStream_t)stream;
#define GD_GO(RPT)                                                                                                         \
  do {                                                                                                                     \
    if (smem > 32 * 1024) cudaFuncSetAttribute(general_delta_scan_kernel<RPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    hb_launch(general_delta_scan_kernel<RPT>, grid, dim3(GD_THREADS), smem, s, a);                                         \
  } while (0)
  if (rpt == 4) GD_GO(4); else if (rpt == 8) GD_GO(8); else if (rpt == 16) GD_GO(16); else GD_GO(32);
#undef GD_GO
  HB_CHECK_LAUNCH("general_delta_scan");
  return 0;
}
