// A sublayer's result joins the residual stream through a gate and a norm of its own:
//
//   v = y * sigmoid(z + b)                          z: a product of the sublayer's input, b a vector (both optional)
//   x <- x + v / sqrt(mean(v^2) + eps) * w          the RMS norm of the result, then the sum
//   h = x / sqrt(mean(x^2) + eps2) * w2             optional: the norm the next sublayer begins with (w2 null: h = x)
//
// in one pass over the stream: a CTA per row keeps v, then the new x, in shared memory.  All float; h leaves in the
// activation type.
//
//   hb_gated_norm_residual   the above
//   hb_token_gate            g[t, j] = gelu_tanh(s[t, j]) * table[id_t][col0 + j]: a gate on a row of numbers that
//                            the token's id chooses from a table (the per-layer part of a second embedding)
#include "api.h"
#include "common.cuh"

struct GatedJoinArgs {
  const float* y; int ldy;
  const float* z; int ldz;      // null: no gate
  const float* zb;              // null: no bias on the gate
  const float* w; float eps;
  float* x;
  const float* w2; float eps2;  // the next norm (w2 null: none)
  void* h;                      // null: nothing is handed on
  int D;
};

template <typename T>
__global__ void __launch_bounds__(256) gated_norm_residual_kernel(GatedJoinArgs a) {
  extern __shared__ float row[];   // [D]
  __shared__ float red[32];
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x, D = a.D;
  const float* y = a.y + (size_t)t * a.ldy;
  const float* z = a.z ? a.z + (size_t)t * a.ldz : nullptr;
  float* x = a.x + (size_t)t * D;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float v = y[i];
    if (z) v *= 1.0f / (1.0f + expf(-(z[i] + (a.zb ? a.zb[i] : 0.0f))));
    row[i] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)D + a.eps);
  float s2 = 0.0f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float xn = x[i] + (row[i] * inv) * a.w[i];
    x[i] = xn;
    row[i] = xn;
    s2 = fmaf(xn, xn, s2);
  }
  if (a.h == nullptr) return;
  T* h = (T*)a.h + (size_t)t * D;
  if (a.w2 == nullptr) {
    for (int i = threadIdx.x; i < D; i += blockDim.x) h[i] = from_f32<T>(row[i]);
    return;
  }
  s2 = block_sum(s2, red);
  const float inv2 = 1.0f / sqrtf(s2 / (float)D + a.eps2);
  for (int i = threadIdx.x; i < D; i += blockDim.x) h[i] = from_f32<T>((row[i] * inv2) * a.w2[i]);
}

extern "C" int hb_gated_norm_residual(int dtype, const float* y, int ldy, const float* z, int ldz, const float* zb,
                                      const float* w, float eps, float* x, const float* w2, float eps2, void* h,
                                      int n_rows, int D, void* stream) {
  HB_REQUIRE(n_rows > 0 && D > 0, "gated_norm_residual: sizes must be positive");
  HB_REQUIRE(z != nullptr || zb == nullptr, "gated_norm_residual: a gate's bias needs the gate");
  const size_t smem = (size_t)D * sizeof(float);
  HB_REQUIRE(smem <= 160 * 1024, "gated_norm_residual: rows of %d numbers do not fit a block's shared memory", D);
  GatedJoinArgs a{y, ldy, z, ldz, zb, w, eps, x, w2, eps2, h, D};
  const int threads = D >= 1024 ? 256 : 128;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == HB_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(gated_norm_residual_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    hb_launch(gated_norm_residual_kernel<float>, dim3(n_rows), dim3(threads), smem, s, a);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(gated_norm_residual_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    hb_launch(gated_norm_residual_kernel<bf16>, dim3(n_rows), dim3(threads), smem, s, a);
  }
  HB_CHECK_LAUNCH("gated_norm_residual");
  return 0;
}

// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void token_gate_kernel(const float* __restrict__ s, int lds, const T* __restrict__ table, int ldt, int col0,
                                  const int* __restrict__ ids, T* __restrict__ out, int ldo, int n_tokens, int m, int vocab) {
  pdl_wait();
  pdl_launch();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)n_tokens * m) return;
  const int t = (int)(i / m), j = (int)(i - (long long)t * m);
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const float g = s[(size_t)t * lds + j];
  const float act = 0.5f * g * (1.0f + tanhf(0.79788456080286535588f * (g + 0.044715f * g * g * g)));
  out[(size_t)t * ldo + j] = from_f32<T>(act * to_f32(table[(size_t)id * ldt + col0 + j]));
}

extern "C" int hb_token_gate(int dtype, const float* s, int lds, const void* table, int ldt, int col0, const int* ids,
                             void* out, int ldo, int n_tokens, int m, int vocab, void* stream) {
  HB_REQUIRE(n_tokens > 0 && m > 0 && vocab > 0, "token_gate: sizes must be positive");
  HB_REQUIRE(col0 >= 0 && col0 + m <= ldt, "token_gate: columns %d..%d lie outside the table's rows of %d", col0, col0 + m, ldt);
  const long long blocks = ceil_div_ll((long long)n_tokens * m, 256);
  HB_REQUIRE(blocks < 2147483647LL, "token_gate: too many elements");
  if (dtype == HB_F32)
    hb_launch(token_gate_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, s, lds, (const float*)table,
              ldt, col0, ids, (float*)out, ldo, n_tokens, m, vocab);
  else
    hb_launch(token_gate_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, s, lds, (const bf16*)table,
              ldt, col0, ids, (bf16*)out, ldo, n_tokens, m, vocab);
  HB_CHECK_LAUNCH("token_gate");
  return 0;
}
