// RMS norm in groups: a row of `dim` numbers is cut into `groups` equal consecutive parts, each part is
// divided by its own sqrt(mean(part^2) + eps), and the whole row is multiplied by a weight vector.
// With one group this is the plain RMS norm.  All arithmetic is float; T is the output's storage type.
//
//   hb_group_rmsnorm           out[r] = GN(x[rows[r]] or x[r]) * w                (the norm before the head)
//   hb_group_rmsnorm_residual  x += GN(y + bias) * w; h = x in the activation dtype   (a sublayer's result joins
//                              the stream, and the next sublayer gets its input, in one pass); with a second array
//                              z the normed vector is a * y + b * z (two mixers side by side, summed here)
//   hb_axpby                   y = a * y + b * z                                  (two mixers side by side)
//   hb_bias_glu                out = act(gate + b) * (up + b) from a product's float sums       (a gated feed-forward with biases)
//   hb_tanh_cap                x = cap * tanh(x / cap)                            (a cap on the logits)
#include "api.h"
#include "common.cuh"

// One CTA per row; warps share the groups: a group of n = dim / groups numbers is summed by the warps that
// hold its elements through shared memory (one float per group).
#define GN_MAX_GROUPS 64
template <typename T, bool RESIDUAL>
__global__ void __launch_bounds__(256)
group_rmsnorm_kernel(const float* __restrict__ y, int ldy, const float* __restrict__ z, int ldz, float a, float b,
                     const float* __restrict__ bias, const float* __restrict__ w, float* __restrict__ x, T* __restrict__ out,
                     const int* __restrict__ rows, int dim, int groups, float eps) {
  __shared__ float sums[GN_MAX_GROUPS];
  pdl_wait();
  pdl_launch();
  const int r = blockIdx.x;
  const float* yr = y + (size_t)(rows ? rows[r] : r) * ldy;
  const float* zr = z ? z + (size_t)r * ldz : nullptr;
  auto value = [&](int i) { return (zr ? a * yr[i] + b * zr[i] : yr[i]) + (bias ? bias[i] : 0.0f); };
  const int n = dim / groups;
  for (int g = threadIdx.x; g < groups; g += blockDim.x) sums[g] = 0.0f;
  __syncthreads();
  // a warp walks whole groups when they are short, else the block walks one group after another
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  for (int g = warp; g < groups; g += nwarp) {
    float s = 0.0f;
    for (int i = lane; i < n; i += 32) {
      const float v = value(g * n + i);
      s = fmaf(v, v, s);
    }
    s = warp_sum(s);
    if (lane == 0) sums[g] = s;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float inv = 1.0f / sqrtf(sums[i / n] / (float)n + eps);
    const float v = (value(i) * inv) * w[i];
    if (RESIDUAL) {
      const float nx = x[(size_t)r * dim + i] + v;
      x[(size_t)r * dim + i] = nx;
      if (out) out[(size_t)r * dim + i] = from_f32<T>(nx);
    } else {
      out[(size_t)r * dim + i] = from_f32<T>(v);
    }
  }
}

static int gn_threads(int dim) { return dim >= 2048 ? 256 : dim >= 512 ? 128 : 64; }

extern "C" int hb_group_rmsnorm(int dtype, const float* x, const float* w, void* out, const int* rows, int n_rows, int dim,
                                int groups, float eps, void* stream) {
  HB_REQUIRE(n_rows > 0 && dim > 0, "group_rmsnorm: sizes must be positive");
  HB_REQUIRE(groups >= 1 && groups <= GN_MAX_GROUPS && dim % groups == 0,
             "group_rmsnorm: %d groups must divide the width %d and be at most %d", groups, dim, GN_MAX_GROUPS);
  if (dtype == HB_F32)
    hb_launch(group_rmsnorm_kernel<float, false>, dim3(n_rows), dim3(gn_threads(dim)), 0, (cudaStream_t)stream, x, dim,
              (const float*)nullptr, 0, 1.0f, 0.0f, (const float*)nullptr, w, (float*)nullptr, (float*)out, rows, dim, groups, eps);
  else
    hb_launch(group_rmsnorm_kernel<bf16, false>, dim3(n_rows), dim3(gn_threads(dim)), 0, (cudaStream_t)stream, x, dim,
              (const float*)nullptr, 0, 1.0f, 0.0f, (const float*)nullptr, w, (float*)nullptr, (bf16*)out, rows, dim, groups, eps);
  HB_CHECK_LAUNCH("group_rmsnorm");
  return 0;
}

extern "C" int hb_group_rmsnorm_residual(int dtype, const float* y, int ldy, const float* z, int ldz, float a, float b,
                                         const float* bias, const float* w, float* x, void* h, int n_rows, int dim, int groups,
                                         float eps, void* stream) {
  HB_REQUIRE(n_rows > 0 && dim > 0, "group_rmsnorm_residual: sizes must be positive");
  HB_REQUIRE(groups >= 1 && groups <= GN_MAX_GROUPS && dim % groups == 0,
             "group_rmsnorm_residual: %d groups must divide the width %d and be at most %d", groups, dim, GN_MAX_GROUPS);
  if (dtype == HB_F32)
    hb_launch(group_rmsnorm_kernel<float, true>, dim3(n_rows), dim3(gn_threads(dim)), 0, (cudaStream_t)stream, y, ldy, z, ldz, a, b,
              bias, w, x, (float*)h, (const int*)nullptr, dim, groups, eps);
  else
    hb_launch(group_rmsnorm_kernel<bf16, true>, dim3(n_rows), dim3(gn_threads(dim)), 0, (cudaStream_t)stream, y, ldy, z, ldz, a, b,
              bias, w, x, (bf16*)h, (const int*)nullptr, dim, groups, eps);
  HB_CHECK_LAUNCH("group_rmsnorm_residual");
  return 0;
}

// ---------------------------------------------------------------------------------------------
__global__ void axpby_kernel(float* __restrict__ y, int ldy, float a, const float* __restrict__ z, int ldz, float b, int rows,
                             int cols) {
  pdl_wait();
  pdl_launch();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)rows * cols) return;
  const int r = (int)(i / cols), c = (int)(i % cols);
  y[(size_t)r * ldy + c] = a * y[(size_t)r * ldy + c] + b * z[(size_t)r * ldz + c];
}

extern "C" int hb_axpby(float* y, int ldy, float a, const float* z, int ldz, float b, int rows, int cols, void* stream) {
  HB_REQUIRE(rows > 0 && cols > 0, "axpby: sizes must be positive");
  const long long blocks = ceil_div_ll((long long)rows * cols, 256);
  HB_REQUIRE(blocks < 2147483647LL, "axpby: too many elements");
  hb_launch(axpby_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, y, ldy, a, z, ldz, b, rows, cols);
  HB_CHECK_LAUNCH("axpby");
  return 0;
}

// gu [n_tokens, 2 inter] floats (a product's sums), bias [2 inter] in the same column layout (or null):
// out = act(gate + b_gate) * (up + b_up) in the activation type.  interleave 0: gate columns [0, inter), up columns
// [inter, 2 inter); interleave n: blocks of 2n columns, n gate then n up.
__device__ __forceinline__ float bias_glu_act(float g, int act) {
  return act == HB_ACT_RELU        ? fmaxf(g, 0.0f)
         : act == HB_ACT_GELU_TANH ? 0.5f * g * (1.0f + tanhf(0.79788456080286535588f * (g + 0.044715f * g * g * g)))
         : act == HB_ACT_GELU      ? 0.5f * g * (1.0f + erff(g * 0.70710678118654752440f))
                                   : g / (1.0f + expf(-g));
}
template <typename T>
__global__ void bias_glu_kernel(const float* __restrict__ gu, int ld, const float* __restrict__ bias, T* __restrict__ out, int ldo,
                                int inter, int interleave, int act) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= inter) return;
  int gi = i, ui = inter + i;
  if (interleave > 0) {
    gi = (i / interleave) * (2 * interleave) + (i % interleave);
    ui = gi + interleave;
  }
  const float* row = gu + (size_t)t * ld;
  const float g = row[gi] + (bias ? bias[gi] : 0.0f), u = row[ui] + (bias ? bias[ui] : 0.0f);
  out[(size_t)t * ldo + i] = from_f32<T>(bias_glu_act(g, act) * u);
}

extern "C" int hb_bias_glu(int dtype, const float* gu, int ld, const float* bias, void* out, int ldo, int n_tokens, int inter,
                           int interleave, int act, void* stream) {
  HB_REQUIRE(n_tokens > 0 && inter > 0, "bias_glu: sizes must be positive");
  HB_REQUIRE(interleave == 0 || (interleave > 0 && inter % interleave == 0),
             "bias_glu: intermediate size %d is no multiple of the interleave %d", inter, interleave);
  HB_REQUIRE(n_tokens <= 65535, "bias_glu: at most 65535 tokens per call, got %d", n_tokens);
  HB_REQUIRE(act >= HB_ACT_SILU && act <= HB_ACT_RELU, "bias_glu: unknown activation %d", act);
  dim3 grid(ceil_div(inter, 256), n_tokens);
  if (dtype == HB_F32)
    hb_launch(bias_glu_kernel<float>, grid, dim3(256), 0, (cudaStream_t)stream, gu, ld, bias, (float*)out, ldo, inter, interleave, act);
  else
    hb_launch(bias_glu_kernel<bf16>, grid, dim3(256), 0, (cudaStream_t)stream, gu, ld, bias, (bf16*)out, ldo, inter, interleave, act);
  HB_CHECK_LAUNCH("bias_glu");
  return 0;
}

__global__ void tanh_cap_kernel(float* __restrict__ x, int ld, float cap, int rows, int cols) {
  pdl_wait();
  pdl_launch();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)rows * cols) return;
  const int r = (int)(i / cols), c = (int)(i % cols);
  x[(size_t)r * ld + c] = cap * tanhf(x[(size_t)r * ld + c] / cap);
}

extern "C" int hb_tanh_cap(float* x, int ld, float cap, int rows, int cols, void* stream) {
  HB_REQUIRE(rows > 0 && cols > 0, "tanh_cap: sizes must be positive");
  HB_REQUIRE(cap > 0.0f, "tanh_cap: the cap must be > 0");
  const long long blocks = ceil_div_ll((long long)rows * cols, 256);
  HB_REQUIRE(blocks < 2147483647LL, "tanh_cap: too many elements");
  hb_launch(tanh_cap_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, x, ld, cap, rows, cols);
  HB_CHECK_LAUNCH("tanh_cap");
  return 0;
}
