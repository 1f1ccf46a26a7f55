// What lies between the q/k/v product and attention for a mixer that norms q and k over the whole projection,
// rotates pairs by angles taken from the position, and keeps its values rotated too:
//
//   q <- q / sqrt(mean_all(q^2) + eps) * wq     over all heads of the row at once (likewise k; optional)
//   pair m of the first `rot` channels of every q and k head turns by  p * fqk[m]
//   pair m of all dv channels of every v head turns by                p * fv[m]      (optional)
//   (u, v) -> (u cos a - v sin a, v cos a + u sin a);  pair m is (2m, 2m + 1) ("interleaved") or (m, m + n/2) ("halves")
//
// The product's rows arrive as floats [q: nh x dk | k: nkv x dk | v: nkv x dv]; q leaves in the activation type with
// heads of `hd` channels, k and v go into the paged cache whose heads have `hd` channels as well.  hd >= max(dk, dv):
// channels beyond dk (dv) are written as zeros, so an attention kernel over heads of hd sees the same scores and
// returns the values' channels followed by zeros.  Angles are float products of the integer position and a float
// frequency, sine and cosine are the accurate ones.
//
//   hb_rotate_heads_back    y[t, h, :dv] = a head's attention result turned by -p (pair m by -p * fv[m]), compacted
//                           from heads of hd channels to heads of dv
//   hb_head_gate            y[t, h, :dv] = a head's attention result times sigmoid(g[t, h]) (one number per token and
//                           head; g null: as it is), compacted likewise
#include "api.h"
#include "common.cuh"

struct RotPrepArgs {
  const float* rows; int ld;
  const float* wq; const float* wk; float eps; int whole_norm;
  const float* fqk; int rot; int halves;
  const float* fv;                 // null: values are stored as they are
  const int* tok_seq; const int* tok_pos; const int* seq_pages; int pages_stride;
  void* q_out; int ldq;
  void* kcache; void* vcache;
  int nh, nkv, dk, dv, hd, page_size, write_cache;
};

// own * cos + (-/+ partner) * sin for channel j of a head whose first `rot` channels are rotated
__device__ __forceinline__ float turn_channel(const float* head, const float* w, float inv, int j, int rot, int halves,
                                              const float* freq, float pos, float dir) {
  const float own = head[j] * inv * (w ? w[j] : 1.0f);
  if (j >= rot) return own;
  int m, partner;
  bool first;
  if (halves) {
    const int half = rot >> 1;
    first = j < half;
    m = first ? j : j - half;
    partner = first ? j + half : j - half;
  } else {
    first = (j & 1) == 0;
    m = j >> 1;
    partner = j ^ 1;
  }
  const float other = head[partner] * inv * (w ? w[partner] : 1.0f);
  float s, c;
  sincosf(pos * freq[m], &s, &c);
  s *= dir;
  return first ? own * c - other * s : own * c + other * s;
}

template <typename T>
__global__ void __launch_bounds__(256) qkv_rotary_cache_kernel(RotPrepArgs a) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x, p = a.tok_pos[t];
  const float pos = (float)p;
  const float* q = a.rows + (size_t)t * a.ld;
  const float* k = q + (size_t)a.nh * a.dk;
  const float* v = k + (size_t)a.nkv * a.dk;
  float inv_q = 1.0f, inv_k = 1.0f;
  if (a.whole_norm) {
    const int nq = a.nh * a.dk, nk = a.nkv * a.dk;
    float sq = 0.0f, sk = 0.0f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) sq = fmaf(q[i], q[i], sq);
    for (int i = threadIdx.x; i < nk; i += blockDim.x) sk = fmaf(k[i], k[i], sk);
    sq = block_sum(sq, red);
    sk = block_sum(sk, red);
    inv_q = 1.0f / sqrtf(sq / (float)nq + a.eps);
    inv_k = 1.0f / sqrtf(sk / (float)nk + a.eps);
  }
  T* qo = (T*)a.q_out + (size_t)t * a.ldq;
  for (int i = threadIdx.x; i < a.nh * a.hd; i += blockDim.x) {
    const int h = i / a.hd, j = i - h * a.hd;
    float r = 0.0f;
    if (j < a.dk) r = turn_channel(q + (size_t)h * a.dk, a.wq ? a.wq + (size_t)h * a.dk : nullptr, inv_q, j, a.rot, a.halves, a.fqk, pos, 1.0f);
    qo[i] = from_f32<T>(r);
  }
  if (!a.write_cache) return;
  const int page = a.seq_pages[(size_t)a.tok_seq[t] * a.pages_stride + p / a.page_size];
  const size_t in_page = (size_t)(p % a.page_size);
  for (int i = threadIdx.x; i < a.nkv * a.hd; i += blockDim.x) {
    const int g = i / a.hd, j = i - g * a.hd;
    const size_t at = (((size_t)page * a.nkv + g) * a.page_size + in_page) * a.hd + j;
    float rk = 0.0f, rv = 0.0f;
    if (j < a.dk) rk = turn_channel(k + (size_t)g * a.dk, a.wk ? a.wk + (size_t)g * a.dk : nullptr, inv_k, j, a.rot, a.halves, a.fqk, pos, 1.0f);
    if (j < a.dv) rv = turn_channel(v + (size_t)g * a.dv, nullptr, 1.0f, j, a.fv ? a.dv : 0, a.halves, a.fv, pos, 1.0f);
    ((T*)a.kcache)[at] = from_f32<T>(rk);
    ((T*)a.vcache)[at] = from_f32<T>(rv);
  }
}

extern "C" int hb_qkv_rotary_cache(int dtype, const float* rows, int ld, const float* wq, const float* wk, float eps,
                                   int whole_norm, const float* fqk, int rot, int halves, const float* fv, const int* tok_seq,
                                   const int* tok_pos, const int* seq_pages, int pages_stride, void* q_out, int ldq, void* kcache,
                                   void* vcache, int n_tokens, int nh, int nkv, int dk, int dv, int hd, int page_size,
                                   int write_cache, void* stream) {
  HB_REQUIRE(n_tokens > 0 && nh > 0 && nkv > 0 && dk > 0 && dv > 0 && page_size > 0, "qkv_rotary_cache: sizes must be positive");
  HB_REQUIRE(hd >= dk && hd >= dv, "qkv_rotary_cache: cache heads of %d channels cannot hold keys of %d and values of %d", hd, dk, dv);
  HB_REQUIRE(rot >= 0 && rot <= dk && rot % 2 == 0, "qkv_rotary_cache: %d rotated channels must be even and at most %d", rot, dk);
  HB_REQUIRE(rot == 0 || fqk != nullptr, "qkv_rotary_cache: rotated channels need their frequencies");
  HB_REQUIRE(fv == nullptr || dv % 2 == 0, "qkv_rotary_cache: rotated values need an even size, got %d", dv);
  // a step that stores nothing (it reads another layer's keys and values) brings rows of queries only
  HB_REQUIRE(ld >= nh * dk + (write_cache ? nkv * (dk + dv) : 0) && ldq >= nh * hd, "qkv_rotary_cache: rows are shorter than their heads");
  RotPrepArgs a{rows, ld, wq, wk, eps, whole_norm, fqk, rot, halves, fv, tok_seq, tok_pos, seq_pages, pages_stride, q_out, ldq,
                kcache, vcache, nh, nkv, dk, dv, hd, page_size, write_cache};
  if (dtype == HB_F32)
    hb_launch(qkv_rotary_cache_kernel<float>, dim3(n_tokens), dim3(256), 0, (cudaStream_t)stream, a);
  else
    hb_launch(qkv_rotary_cache_kernel<bf16>, dim3(n_tokens), dim3(256), 0, (cudaStream_t)stream, a);
  HB_CHECK_LAUNCH("qkv_rotary_cache");
  return 0;
}

// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
rotate_heads_back_kernel(const T* __restrict__ att, int ld, int hd, const float* __restrict__ fv, int halves,
                         const int* __restrict__ tok_pos, T* __restrict__ y, int ldy, int nh, int dv) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x;
  const float pos = (float)tok_pos[t];
  const T* ar = att + (size_t)t * ld;
  T* yr = y + (size_t)t * ldy;
  const int half = dv >> 1;
  for (int i = threadIdx.x; i < nh * half; i += blockDim.x) {
    const int h = i / half, m = i - h * half;
    const int j0 = halves ? m : 2 * m, j1 = halves ? m + half : 2 * m + 1;
    const float u = to_f32(ar[(size_t)h * hd + j0]), w = to_f32(ar[(size_t)h * hd + j1]);
    float s = 0.0f, c = 1.0f;
    if (fv) sincosf(pos * fv[m], &s, &c);
    // the turn by -a
    yr[(size_t)h * dv + j0] = from_f32<T>(u * c + w * s);
    yr[(size_t)h * dv + j1] = from_f32<T>(w * c - u * s);
  }
}

extern "C" int hb_rotate_heads_back(int dtype, const void* att, int ld, int hd, const float* fv, int halves, const int* tok_pos,
                                    void* y, int ldy, int n_tokens, int nh, int dv, void* stream) {
  HB_REQUIRE(n_tokens > 0 && nh > 0 && dv > 0 && hd >= dv, "rotate_heads_back: sizes must be positive and heads wide enough");
  HB_REQUIRE(dv % 2 == 0, "rotate_heads_back: values of %d channels have no pairs", dv);
  if (dtype == HB_F32)
    hb_launch(rotate_heads_back_kernel<float>, dim3(n_tokens), dim3(128), 0, (cudaStream_t)stream, (const float*)att, ld, hd, fv,
              halves, tok_pos, (float*)y, ldy, nh, dv);
  else
    hb_launch(rotate_heads_back_kernel<bf16>, dim3(n_tokens), dim3(128), 0, (cudaStream_t)stream, (const bf16*)att, ld, hd, fv,
              halves, tok_pos, (bf16*)y, ldy, nh, dv);
  HB_CHECK_LAUNCH("rotate_heads_back");
  return 0;
}

// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
head_gate_kernel(const T* __restrict__ att, int ld, int hd, const float* __restrict__ gate, int ldg, T* __restrict__ y, int ldy,
                 int nh, int dv) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x;
  const T* ar = att + (size_t)t * ld;
  T* yr = y + (size_t)t * ldy;
  for (int i = threadIdx.x; i < nh * dv; i += blockDim.x) {
    const int h = i / dv, j = i - h * dv;
    const float g = gate ? 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + h])) : 1.0f;
    yr[i] = from_f32<T>(to_f32(ar[(size_t)h * hd + j]) * g);
  }
}

extern "C" int hb_head_gate(int dtype, const void* att, int ld, int hd, const float* gate, int ldg, void* y, int ldy,
                            int n_tokens, int nh, int dv, void* stream) {
  HB_REQUIRE(n_tokens > 0 && nh > 0 && dv > 0 && hd >= dv, "head_gate: sizes must be positive and heads wide enough");
  if (dtype == HB_F32)
    hb_launch(head_gate_kernel<float>, dim3(n_tokens), dim3(128), 0, (cudaStream_t)stream, (const float*)att, ld, hd, gate, ldg,
              (float*)y, ldy, nh, dv);
  else
    hb_launch(head_gate_kernel<bf16>, dim3(n_tokens), dim3(128), 0, (cudaStream_t)stream, (const bf16*)att, ld, hd, gate, ldg,
              (bf16*)y, ldy, nh, dv);
  HB_CHECK_LAUNCH("head_gate");
  return 0;
}
