// A routed feed-forward: every token goes through `top` of E small feed-forwards.
//
//   z = R h (float);  s = softmax(z) over all E experts;  the `top` largest s are chosen
//   weights: the chosen s themselves, or (renorm) divided by their sum
//   y = sum over the chosen e of weight_e * Down_e act(Up_e h)      act: gelu (erf form) or silu
// Options of the router: s = sigmoid(z) instead of the softmax; the experts as `groups` equal groups
// of neighbours, a group's score being the sum of its `group_top` largest s, with only the experts of
// the `keep` best groups open to the choice (ties between groups, as between experts, go to the
// lower index); a factor on every weight.  Option of the experts: a gated form
// Down_e (act(Gate_e h) * (Up_e h)) whose first matrix has 2F rows per expert: `gated` 2: the rows of
// Gate_e and Up_e in turn in groups of 8 (8 gate rows, the 8 up rows of the same channels, ...: the layout
// of the dense gated feed-forward, so that a thread of a tensor-core tile holds both halves of a
// channel); `gated` 1: all gate rows, then all up rows (any F; the few-token kernel only).
//
// Three launches, all reading the choice from device memory (nothing of it is known to the host, so
// a recorded step can be replayed): the router with softmax and choice; the chosen experts' first
// product with the activation; their second product with the weighted sum.  A warp computes one
// output number from one weight row read along its length, which is what a step of few tokens
// wants: every weight row of a chosen expert is read once per token that chose it.
#include "api.h"
#include "common.cuh"

#define MOE_WARPS 4
#define MOE_ROUTE_WARPS 8

// A warp's dot product of two rows of n numbers: 16 bytes per lane and step where the rows allow it.
__device__ __forceinline__ float warp_dot(const float* a, const float* w, int n, int lane) {
  float dot = 0.0f;
  if ((n & 3) == 0 && ((((uintptr_t)a) | ((uintptr_t)w)) & 15) == 0) {
    const float4* a4 = reinterpret_cast<const float4*>(a);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    for (int i = lane; i < (n >> 2); i += 32) {
      const float4 x = a4[i], y = w4[i];
      dot = fmaf(x.x, y.x, dot); dot = fmaf(x.y, y.y, dot); dot = fmaf(x.z, y.z, dot); dot = fmaf(x.w, y.w, dot);
    }
  } else {
    for (int i = lane; i < n; i += 32) dot = fmaf(a[i], w[i], dot);
  }
  return warp_sum(dot);
}
__device__ __forceinline__ float warp_dot(const bf16* a, const bf16* w, int n, int lane) {
  float dot = 0.0f;
  if ((n & 7) == 0 && ((((uintptr_t)a) | ((uintptr_t)w)) & 15) == 0) {
    const uint4* a4 = reinterpret_cast<const uint4*>(a);
    const uint4* w4 = reinterpret_cast<const uint4*>(w);
    for (int i = lane; i < (n >> 3); i += 32) {
      const uint4 x = a4[i], y = w4[i];
      const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&x);
      const __nv_bfloat162* yp = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 xf = __bfloat1622float2(xp[j]), yf = __bfloat1622float2(yp[j]);
        dot = fmaf(xf.x, yf.x, dot);
        dot = fmaf(xf.y, yf.y, dot);
      }
    }
  } else {
    for (int i = lane; i < n; i += 32) dot = fmaf(__bfloat162float(a[i]), __bfloat162float(w[i]), dot);
  }
  return warp_sum(dot);
}

// One block per token: its warps share the experts' dot products, the first warp then takes the
// scores, the groups and the choice.
template <typename T>
__global__ void __launch_bounds__(MOE_ROUTE_WARPS * 32)
moe_route_kernel(const T* __restrict__ h, int ld, const T* __restrict__ wr, int* __restrict__ ids, float* __restrict__ wts,
                 int n_tokens, int D, int E, int top, int renorm, int sigmoid, int groups, int keep, int group_top,
                 float wscale) {
  extern __shared__ float sh[];  // [E] scores, [groups] group scores
  pdl_wait();
  pdl_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  float* s = sh;
  float* gs = sh + E;
  const T* hr = h + (size_t)t * ld;
  for (int e = warp; e < E; e += MOE_ROUTE_WARPS) {
    const float dot = warp_dot(hr, wr + (size_t)e * D, D, lane);
    if (lane == 0) s[e] = dot;
  }
  __syncthreads();
  if (warp != 0) return;
  if (sigmoid) {
    for (int e = lane; e < E; e += 32) s[e] = 1.0f / (1.0f + expf(-s[e]));
  } else {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, s[e]);
    mx = warp_max(mx);
    float sum = 0.0f;
    for (int e = lane; e < E; e += 32) sum += expf(s[e] - mx);
    sum = warp_sum(sum);
    for (int e = lane; e < E; e += 32) s[e] = expf(s[e] - mx) / sum;
  }
  __syncwarp();
  if (groups > 1) {
    const int size = E / groups;
    // a group's score: the sum of those of its scores that fewer than group_top others beat
    for (int g = lane; g < groups; g += 32) {
      const float* sg = s + g * size;
      float acc = 0.0f;
      for (int i = 0; i < size; ++i) {
        int beaten = 0;
        for (int j = 0; j < size; ++j) beaten += (sg[j] > sg[i] || (sg[j] == sg[i] && j < i)) ? 1 : 0;
        if (beaten < group_top) acc += sg[i];
      }
      gs[g] = acc;
    }
    __syncwarp();
    // experts of groups that `keep` or more others beat leave the choice (scores are >= 0; -3 never wins)
    for (int e = lane; e < E; e += 32) {
      const int g = e / size;
      int beaten = 0;
      for (int j = 0; j < groups; ++j) beaten += (gs[j] > gs[g] || (gs[j] == gs[g] && j < g)) ? 1 : 0;
      if (beaten >= keep) s[e] = -3.0f;
    }
    __syncwarp();
  }
  float chosen_sum = 0.0f;
  for (int r = 0; r < top; ++r) {
    float best = -1.0f;
    int bi = E;
    for (int e = lane; e < E; e += 32)
      if (s[e] > best) { best = s[e]; bi = e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) {
      ids[(size_t)t * top + r] = bi;
      wts[(size_t)t * top + r] = best * wscale;
      s[bi] = -2.0f;  // taken
    }
    chosen_sum += best;
    __syncwarp();
  }
  if (renorm && lane == 0)
    for (int r = 0; r < top; ++r) wts[(size_t)t * top + r] /= chosen_sum;
}

extern "C" int hb_moe_route(int dtype, const void* h, int ld, const void* w_router, int* ids, float* weights, int n_tokens,
                            int D, int E, int top, int renorm, int sigmoid, int groups, int keep, int group_top,
                            float wscale, void* stream) {
  HB_REQUIRE(n_tokens > 0 && D > 0 && E > 0 && top > 0 && top <= E, "moe_route: bad sizes (experts %d, top %d)", E, top);
  HB_REQUIRE(groups >= 1 && E % groups == 0 && keep >= 1 && keep <= groups && group_top >= 1,
             "moe_route: %d experts in %d groups of which %d are kept", E, groups, keep);
  HB_REQUIRE(top <= (E / groups) * keep, "moe_route: %d groups of %d experts cannot give %d choices", keep, E / groups, top);
  const size_t smem = (size_t)(E + groups) * sizeof(float);
  HB_REQUIRE(smem <= 48 * 1024, "moe_route: %d experts exceed what a block keeps in shared memory", E);
  dim3 grid(n_tokens);
  if (dtype == HB_F32)
    hb_launch(moe_route_kernel<float>, grid, dim3(MOE_ROUTE_WARPS * 32), smem, (cudaStream_t)stream, (const float*)h, ld, (const float*)w_router, ids, weights, n_tokens, D, E, top, renorm, sigmoid, groups, keep, group_top, wscale);
  else
    hb_launch(moe_route_kernel<bf16>, grid, dim3(MOE_ROUTE_WARPS * 32), smem, (cudaStream_t)stream, (const bf16*)h, ld, (const bf16*)w_router, ids, weights, n_tokens, D, E, top, renorm, sigmoid, groups, keep, group_top, wscale);
  HB_CHECK_LAUNCH("moe_route");
  return 0;
}

// A gated expert's hidden value from its two products.  The clamped form (HB_ACT_SWISH_CLAMP, with a limit L):
// g' = min(g, L), v' = clamp(v, -L, L), g' sigmoid(1.702 g') (v' + 1); every other activation: act(g) v.
__device__ __forceinline__ float moe_act(float z, int act);
__device__ __forceinline__ float moe_glu(float g, float v, int act, float limit) {
  if (act == HB_ACT_SWISH_CLAMP) {
    g = fminf(g, limit);
    v = fminf(fmaxf(v, -limit), limit);
    return (g / (1.0f + expf(-HB_SWISH_CLAMP_SLOPE * g))) * (v + 1.0f);
  }
  return moe_act(g, act) * v;
}
__device__ __forceinline__ float moe_act(float z, int act) {
  if (act == HB_ACT_GELU) return 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
  if (act == HB_ACT_GELU_TANH) return 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
  return z / (1.0f + expf(-z));
}

// mid[(t*top + r), f] = act(Up_e[f, :] . h[t, :]),  e = ids[t, r]; gated: act(gate row f . h) * (up row f . h) of
// the expert's 2F rows.  One warp per output.
template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_up_kernel(const T* __restrict__ h, int ld, const T* __restrict__ up, const int* __restrict__ ids, T* __restrict__ mid,
              int D, int F, int top, int act, int gated, float limit) {
  pdl_wait();
  pdl_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int f = blockIdx.y * MOE_WARPS + warp, u = blockIdx.x;  // u = t*top + r
  if (f >= F) return;
  const int e = ids[u];
  const T* hr = h + (size_t)(u / top) * ld;
  if (gated) {
    const int grow = gated == 2 ? (f >> 3) * 16 + (f & 7) : f, urow = gated == 2 ? grow + 8 : F + f;
    const T* w = up + (size_t)e * 2 * F * D;
    const float g = warp_dot(hr, w + (size_t)grow * D, D, lane), v = warp_dot(hr, w + (size_t)urow * D, D, lane);
    if (lane == 0) mid[(size_t)u * F + f] = from_f32<T>(moe_glu(g, v, act, limit));
    return;
  }
  const T* w = up + ((size_t)e * F + f) * D;
  const float dot = warp_dot(hr, w, D, lane);
  if (lane == 0) mid[(size_t)u * F + f] = from_f32<T>(moe_act(dot, act));
}

// y[t, d] (+)= sum_r wts[t, r] * Down_e[d, :] . mid[(t*top + r), :].  One warp per output.
template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_down_kernel(const T* __restrict__ mid, const T* __restrict__ down, const int* __restrict__ ids, const float* __restrict__ wts,
                float* __restrict__ y, int ldy, int D, int F, int top, int accumulate) {
  pdl_wait();
  pdl_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int d = blockIdx.y * MOE_WARPS + warp, t = blockIdx.x;
  if (d >= D) return;
  float acc = 0.0f;
  for (int r = 0; r < top; ++r) {
    const int u = t * top + r;
    const T* w = down + ((size_t)ids[u] * D + d) * F;
    const T* m = mid + (size_t)u * F;
    acc = fmaf(wts[u], warp_dot(m, w, F, lane), acc);
  }
  if (lane == 0) {
    float* o = y + (size_t)t * ldy + d;
    *o = accumulate ? *o + acc : acc;
  }
}

extern "C" int hb_moe_experts(int dtype, const void* h, int ld, const void* up, const void* down, const int* ids,
                              const float* weights, void* mid, float* y, int ldy, int n_tokens, int D, int F, int top,
                              int act, int gated, float act_limit, int accumulate, void* stream) {
  HB_REQUIRE(n_tokens > 0 && D > 0 && F > 0 && top > 0, "moe_experts: sizes must be positive");
  HB_REQUIRE(act != HB_ACT_SWISH_CLAMP || gated, "moe_experts: the clamped activation is a gated expert's");
  HB_REQUIRE((long long)n_tokens * top < 2147483647LL && ceil_div(F, MOE_WARPS) <= 65535 && ceil_div(D, MOE_WARPS) <= 65535,
             "moe_experts: too many (token, choice) pairs or channels");
  cudaStream_t s = (cudaStream_t)stream;
  dim3 g1(n_tokens * top, ceil_div(F, MOE_WARPS)), g2(n_tokens, ceil_div(D, MOE_WARPS));
  if (dtype == HB_F32) {
    hb_launch(moe_up_kernel<float>, g1, dim3(MOE_WARPS * 32), 0, s, (const float*)h, ld, (const float*)up, ids, (float*)mid, D, F, top, act, gated, act_limit);
    hb_launch(moe_down_kernel<float>, g2, dim3(MOE_WARPS * 32), 0, s, (const float*)mid, (const float*)down, ids, weights, y, ldy, D, F, top, accumulate);
  } else {
    hb_launch(moe_up_kernel<bf16>, g1, dim3(MOE_WARPS * 32), 0, s, (const bf16*)h, ld, (const bf16*)up, ids, (bf16*)mid, D, F, top, act, gated, act_limit);
    hb_launch(moe_down_kernel<bf16>, g2, dim3(MOE_WARPS * 32), 0, s, (const bf16*)mid, (const bf16*)down, ids, weights, y, ldy, D, F, top, accumulate);
  }
  HB_CHECK_LAUNCH("moe_experts");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Steps of many tokens (prompts), bfloat16: the (token, choice) pairs are grouped by expert on the
// device and each expert's pairs go through the tensor cores in tiles of 128 rows x 128 outputs, so an
// expert's matrices are read once per 128 pairs instead of once per pair.
//   hb_moe_group:   counts per expert, where each expert's pairs and tiles begin, the pairs listed by expert
//   grouped product (mma.sync m16n8k16): rows gathered through the list; first product with the
//                   activation into mid[pair], second product into part[pair] (float)
//   combine:        y[t] (+)= sum_r weights[t, r] * part[t * top + r]
// Which place a pair gets inside its expert's list depends on the order in which threads arrive; a
// pair's own numbers do not depend on its place, so the result is the same bits every time.
#include "mma_utils.cuh"

#define MG_TM 128
#define MG_TN 128
#define MG_TK 32
#define MG_THREADS 256
#define MG_MAX_EXPERTS 1024

__global__ void __launch_bounds__(1024)
moe_group_kernel(const int* __restrict__ ids, int n_pairs, int E, int* __restrict__ pair_off, int* __restrict__ tile_off,
                 int* __restrict__ list) {
  __shared__ int cnt[MG_MAX_EXPERTS], off[MG_MAX_EXPERTS + 1];
  pdl_wait();
  pdl_launch();
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int u = threadIdx.x; u < n_pairs; u += blockDim.x) atomicAdd(&cnt[ids[u]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int p = 0, tl = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = p;
      pair_off[e] = p;
      tile_off[e] = tl;
      p += cnt[e];
      tl += (cnt[e] + MG_TM - 1) / MG_TM;
    }
    off[E] = p;
    pair_off[E] = p;
    tile_off[E] = tl;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int u = threadIdx.x; u < n_pairs; u += blockDim.x) {
    const int e = ids[u];
    list[off[e] + atomicAdd(&cnt[e], 1)] = u;
  }
}

// C[pair, n] = sum_k A[row(pair), k] * W[e][n][k] for the pairs of tile blockIdx.x of its expert.
// UP: row(pair) = pair / top of h, C = act(.) as bfloat16 into mid[pair]; else row(pair) = pair of mid, C float into part[pair].
// UP and gated: W has 2F rows per expert, gate and up in turn in groups of 8, and a thread's columns of fragment nt (even: gate)
// and nt + 1 (up) are the two halves of its channels.
template <bool UP>
__global__ void __launch_bounds__(MG_THREADS)
moe_grouped_gemm_kernel(const bf16* __restrict__ A, int lda, const bf16* __restrict__ W, void* __restrict__ C, int ldc,
                        const int* __restrict__ pair_off, const int* __restrict__ tile_off, const int* __restrict__ list, int E,
                        int N, int K, int top, int act, int gated, float limit) {
  __shared__ __align__(16) bf16 AW[2][(MG_TM + MG_TN) * (MG_TK + 8)];      // per buffer: the A tile, then the W tile
  __shared__ int rows[MG_TM];
  pdl_wait();
  pdl_launch();
  const int tile = blockIdx.x;
  if (tile >= tile_off[E]) return;
  int e = 0;
  while (tile >= tile_off[e + 1]) ++e;
  const int first = pair_off[e] + (tile - tile_off[e]) * MG_TM, end = pair_off[e + 1];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int wm = (warp & 3) * 32, wn = (warp >> 2) * 64;      // this warp's 32 rows x 64 outputs of the tile
  if (tid < MG_TM) rows[tid] = first + tid < end ? list[first + tid] : -1;
  __syncthreads();
  const int n0 = blockIdx.y * MG_TN;
  const bf16* We = W + (size_t)e * N * K;

  // 128 rows x 4 pieces of 16 bytes for A and as many for W: 1,024 pieces, 4 per thread, the same (row, piece)
  // in every k slab, so where each comes from is worked out once
  constexpr int PIECES = 2 * MG_TM * (MG_TK / 8) / MG_THREADS;
  const bf16* src0[PIECES];
  int dst0[PIECES], kc[PIECES];
#pragma unroll
  for (int q = 0; q < PIECES; ++q) {
    const int i = tid + q * MG_THREADS;
    const bool isw = i >= MG_TM * (MG_TK / 8);
    const int j = isw ? i - MG_TM * (MG_TK / 8) : i;
    const int r = j / (MG_TK / 8), c = (j % (MG_TK / 8)) * 8;
    kc[q] = c;
    dst0[q] = (isw ? MG_TM * (MG_TK + 8) : 0) + r * (MG_TK + 8) + c;      // As and Ws of a buffer lie one after the other below
    src0[q] = nullptr;
    if (isw) {
      if (n0 + r < N) src0[q] = We + (size_t)(n0 + r) * K + c;
    } else if (rows[r] >= 0) {
      src0[q] = A + (size_t)(UP ? rows[r] / top : rows[r]) * lda + c;
    }
  }
  auto load = [&](int buf, int k0) {
    bf16* base = &AW[buf][0];
#pragma unroll
    for (int q = 0; q < PIECES; ++q) {
      bf16* dst = base + dst0[q];
      if (src0[q] && k0 + kc[q] < K) cp_async16(dst, src0[q] + k0);
      else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    cp_async_commit();
  };

  float acc[2][8][4];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[m][i][c] = 0.0f;
  const int nk = (K + MG_TK - 1) / MG_TK;
  load(0, 0);
  for (int kb = 0; kb < nk; ++kb) {
    if (kb + 1 < nk) {
      load((kb + 1) & 1, (kb + 1) * MG_TK);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int buf = kb & 1;
#pragma unroll
    for (int ks = 0; ks < MG_TK / 16; ++ks) {
      unsigned a[2][4];
#pragma unroll
      for (int m = 0; m < 2; ++m)
        ldmatrix_x4(a[m][0], a[m][1], a[m][2], a[m][3], &AW[buf][(wm + m * 16 + (lane & 15)) * (MG_TK + 8) + ks * 16 + (lane >> 4) * 8]);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        unsigned b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, &AW[buf][(MG_TM + wn + np * 16 + (lane & 7) + ((lane >> 4) << 3)) * (MG_TK + 8) + ks * 16 + ((lane >> 3) & 1) * 8]);
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          mma16816(acc[m][2 * np], a[m][0], a[m][1], a[m][2], a[m][3], b0, b1);
          mma16816(acc[m][2 * np + 1], a[m][0], a[m][1], a[m][2], a[m][3], b2, b3);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int pair = rows[wm + m * 16 + g + half * 8];
      if (pair < 0) continue;
      if (UP && gated) {
#pragma unroll
        for (int nt = 0; nt < 8; nt += 2)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int n = n0 + wn + nt * 8 + 2 * t + c;      // a gate column; its up column is n + 8 (N is a multiple of 16)
            if (n >= N) continue;
            ((bf16*)C)[(size_t)pair * ldc + ((n0 + wn + nt * 8) >> 1) + 2 * t + c] =
                __float2bfloat16_rn(moe_glu(acc[m][nt][half * 2 + c], acc[m][nt + 1][half * 2 + c], act, limit));
          }
        continue;
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int n = n0 + wn + nt * 8 + 2 * t + c;
          if (n >= N) continue;
          const float v = acc[m][nt][half * 2 + c];
          if (UP) ((bf16*)C)[(size_t)pair * ldc + n] = __float2bfloat16_rn(moe_act(v, act));
          else ((float*)C)[(size_t)pair * ldc + n] = v;
        }
    }
}

// slot: where each pair's row lies in `part` (null: at the pair's own index)
__global__ void moe_combine_kernel(const float* __restrict__ part, const float* __restrict__ wts, float* __restrict__ y, int ldy,
                                   int D, int top, int accumulate, const int* __restrict__ slot) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.y, d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= D) return;
  float acc = 0.0f;
  for (int r = 0; r < top; ++r) {
    const size_t u = (size_t)t * top + r;
    acc = fmaf(wts[u], part[(slot ? (size_t)slot[u] : u) * D + d], acc);
  }
  float* o = y + (size_t)t * ldy + d;
  *o = accumulate ? *o + acc : acc;
}

extern "C" long long hb_moe_grouped_scratch_ints(int n_tokens, int E, int top) {
  return 2LL * (E + 1) + (long long)n_tokens * top;
}

// scratch: hb_moe_grouped_scratch_ints ints; mid [T * top, F] bfloat16; part [T * top, D] floats.
extern "C" int hb_moe_experts_grouped_bf16(const void* h, int ld, const void* up, const void* down, const int* ids,
                                           const float* weights, int* scratch, void* mid, float* part, float* y, int ldy,
                                           int n_tokens, int D, int E, int F, int top, int act, int gated,
                                           float act_limit, int accumulate, void* stream) {
  HB_REQUIRE(n_tokens > 0 && D > 0 && E > 0 && F > 0 && top > 0, "moe_experts_grouped: sizes must be positive");
  HB_REQUIRE(E <= MG_MAX_EXPERTS, "moe_experts_grouped: at most %d experts", MG_MAX_EXPERTS);
  HB_REQUIRE(D % 8 == 0 && F % 8 == 0 && ld % 8 == 0, "moe_experts_grouped: widths must be multiples of 8");
  HB_REQUIRE(gated == 0 || gated == 2, "moe_experts_grouped: gated experts need their gate and up rows in groups of 8");
  HB_REQUIRE(act != HB_ACT_SWISH_CLAMP || gated, "moe_experts_grouped: the clamped activation is a gated expert's");
  HB_REQUIRE(n_tokens <= 65535, "moe_experts_grouped: at most 65535 tokens per call");
  const int n_pairs = n_tokens * top;
  int* pair_off = scratch;
  int* tile_off = scratch + (E + 1);
  int* list = scratch + 2 * (E + 1);
  cudaStream_t s = (cudaStream_t)stream;
  hb_launch(moe_group_kernel, dim3(1), dim3(1024), 0, s, ids, n_pairs, E, pair_off, tile_off, list);
  const int max_tiles = ceil_div(n_pairs, MG_TM) + E;
  const int n_up = gated ? 2 * F : F;      // rows of an expert's first matrix
  hb_launch(moe_grouped_gemm_kernel<true>, dim3(max_tiles, ceil_div(n_up, MG_TN)), dim3(MG_THREADS), 0, s, (const bf16*)h, ld, (const bf16*)up,
            mid, F, (const int*)pair_off, (const int*)tile_off, (const int*)list, E, n_up, D, top, act, gated, act_limit);
  hb_launch(moe_grouped_gemm_kernel<false>, dim3(max_tiles, ceil_div(D, MG_TN)), dim3(MG_THREADS), 0, s, (const bf16*)mid, F,
            (const bf16*)down, (void*)part, D, (const int*)pair_off, (const int*)tile_off, (const int*)list, E, D, F, top, act, 0, 0.0f);
  hb_launch(moe_combine_kernel, dim3(ceil_div(D, 256), n_tokens), dim3(256), 0, s, (const float*)part, weights, y, ldy, D, top, accumulate, (const int*)nullptr);
  HB_CHECK_LAUNCH("moe_experts_grouped");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Long prompts, gated experts with silu (act_limit 0) or the clamped activation (act_limit L > 0), bfloat16: the grouped
// products on tcgen05.  The pairs are sorted by
// expert into a buffer in which every expert's run is padded to whole tiles of 128 rows, so that a tile of the
// tensor-memory product (gemm_tcgen05.cu, grouped mode) belongs to one expert:
//   sort:     counts per expert, padded offsets, slot[pair] = its row, tile_expert[tile], rows in use
//   gather:   sorted[slot[pair]] = h[pair / top]
//   product:  mid = silu(gate) * up of sorted x W1_e (the dense feed-forward's fused epilogue)
//   product:  part = mid x W2_e (float)
//   combine:  y[t] (+)= sum_r weights[t, r] * part[slot[t * top + r]]
// Rows of padding are computed and never read.  A pair's numbers do not depend on its place.
__global__ void __launch_bounds__(1024)
moe_sort_padded_kernel(const int* __restrict__ ids, int n_pairs, int E, int* __restrict__ slot, int* __restrict__ tile_expert,
                       int* __restrict__ rows_used, int max_tiles) {
  __shared__ int cnt[MG_MAX_EXPERTS], off[MG_MAX_EXPERTS];
  pdl_wait();
  pdl_launch();
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int u = threadIdx.x; u < n_pairs; u += blockDim.x) atomicAdd(&cnt[ids[u]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int tl = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = tl * 128;
      const int n = (cnt[e] + 127) / 128;
      for (int i = 0; i < n && tl + i < max_tiles; ++i) tile_expert[tl + i] = e;
      tl += n;
    }
    *rows_used = (tl < max_tiles ? tl : max_tiles) * 128;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int u = threadIdx.x; u < n_pairs; u += blockDim.x) {
    const int e = ids[u];
    slot[u] = off[e] + atomicAdd(&cnt[e], 1);
  }
}

__global__ void moe_gather_rows_kernel(const bf16* __restrict__ h, int ld, const int* __restrict__ slot, bf16* __restrict__ sorted,
                                       int D8, int top) {
  pdl_wait();
  pdl_launch();
  const int u = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(h + (size_t)(u / top) * ld);
  uint4* dst = reinterpret_cast<uint4*>(sorted + (size_t)slot[u] * D8 * 8);
  for (int i = threadIdx.x; i < D8; i += blockDim.x) dst[i] = src[i];
}

// Rows of the sorted, padded buffers for n_tokens * top pairs of E experts.
extern "C" int hb_moe_experts_tc_rows(int n_tokens, int E, int top) {
  const long long tiles = ((long long)n_tokens * top + 127) / 128 + E;
  return tiles * 128 > 2147483647LL ? -1 : (int)(tiles * 128);
}

// up [E, 2F, D] with gate and up rows in groups of 8; ints: n_tokens * top + rows / 128 + 1; sorted [rows, D] and
// mid [rows, F] bfloat16, part [rows, D] floats, with rows = hb_moe_experts_tc_rows(...).
extern "C" int hb_moe_experts_tc_bf16(const void* h, int ld, const void* up, const void* down, const int* ids,
                                      const float* weights, int* ints, void* sorted, void* mid, float* part, float* y, int ldy,
                                      int n_tokens, int D, int E, int F, int top, float act_limit, int accumulate,
                                      int* error_flag, void* stream) {
  HB_REQUIRE(n_tokens > 0 && D > 0 && E > 0 && F > 0 && top > 0, "moe_experts_tc: sizes must be positive");
  HB_REQUIRE(E <= MG_MAX_EXPERTS, "moe_experts_tc: at most %d experts", MG_MAX_EXPERTS);
  HB_REQUIRE(D % 8 == 0 && F % 8 == 0 && ld % 8 == 0 && ((uintptr_t)h & 15) == 0, "moe_experts_tc: widths must be multiples of 8, rows 16-byte aligned");
  HB_REQUIRE(n_tokens <= 65535, "moe_experts_tc: at most 65535 tokens per call");
  const int rows = hb_moe_experts_tc_rows(n_tokens, E, top);
  HB_REQUIRE(rows > 0, "moe_experts_tc: too many pairs");
  const int n_pairs = n_tokens * top, max_tiles = rows / 128;
  int* slot = ints;
  int* tile_expert = ints + n_pairs;
  int* rows_used = tile_expert + max_tiles;
  cudaStream_t s = (cudaStream_t)stream;
  hb_launch(moe_sort_padded_kernel, dim3(1), dim3(1024), 0, s, ids, n_pairs, E, slot, tile_expert, rows_used, max_tiles);
  hb_launch(moe_gather_rows_kernel, dim3(n_pairs), dim3(D / 8 >= 128 ? 128 : 64), 0, s, (const bf16*)h, ld, (const int*)slot,
            (bf16*)sorted, D / 8, top);
  HB_CHECK_LAUNCH("moe_experts_tc (sort, gather)");
  int rc = hb_gemm_tcgen05_grouped_bf16(sorted, D, up, D, mid, F, rows, 2 * F, D, E, HB_EPI_SWIGLU, act_limit, rows_used,
                                        tile_expert, error_flag, stream);
  if (rc) return rc;
  rc = hb_gemm_tcgen05_grouped_bf16(mid, F, down, F, part, D, rows, D, F, E, HB_EPI_STORE_F32, 0.0f, rows_used, tile_expert,
                                    error_flag, stream);
  if (rc) return rc;
  hb_launch(moe_combine_kernel, dim3(ceil_div(D, 256), n_tokens), dim3(256), 0, s, (const float*)part, weights, y, ldy, D, top,
            accumulate, (const int*)slot);
  HB_CHECK_LAUNCH("moe_experts_tc (combine)");
  return 0;
}
