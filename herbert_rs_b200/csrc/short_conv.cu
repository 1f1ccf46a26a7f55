// A short causal convolution over time, channel by channel, whose last inputs are a sequence's state;
// and an embedding to which a row chosen by (previous token, token) is added, whose previous token is state too.
//
//   conv:   c_t = sum_j w[:, j] * u_{t - taps + 1 + j}      (w [channels, taps]; the last column weighs u_t itself;
//                                                            zeros before the sequence's start)
//           out_t = u_t + c_t (add_input)  or  c_t,  then silu if asked
//   state:  [slots, taps - 1, channels] floats: the inputs u of the sequence's last taps - 1 positions, zero when
//           the slot is handed out.  A step reads them for its first tokens and leaves its own last inputs there,
//           so a prompt in one step, in pieces or token by token convolves the same numbers.
//
//   pair embedding:  x_t = E[id_t] * scale + P[(id_{t-1} * a + id_t * b) mod n],  P's row n for a sequence's first token;
//           the id before a step's first token is the int the step before left in the sequence's slot.
#include "api.h"
#include "common.cuh"

#define SC_THREADS 128
#define SC_TOKENS 64   // most tokens per CTA; a CTA takes at least taps - 1, so that only a sequence's first CTA reads its state

template <typename TO>
__global__ void __launch_bounds__(SC_THREADS)
short_conv_kernel(const float* __restrict__ in, int ld_in, const float* __restrict__ w, float* __restrict__ state,
                  const int* __restrict__ seq_slot, const int* __restrict__ seq_start, const int* __restrict__ seq_pos0,
                  TO* __restrict__ out, int ldo, int C, int taps, int add_input, int act_silu, int span) {
  pdl_wait();
  pdl_launch();
  const int c = blockIdx.x * SC_THREADS + threadIdx.x;
  const int b = blockIdx.z;
  const int t0 = seq_start[b], n = seq_start[b + 1] - t0;
  const int lo = blockIdx.y * span;
  if (lo >= n || c >= C) return;
  const int hi = lo + span < n ? lo + span : n;
  const int back = taps - 1;
  const int pos0 = seq_pos0[b];
  float* st = state ? state + (size_t)seq_slot[b] * back * C + c : nullptr;
  const float* wr = w + (size_t)c * taps;
  for (int i = lo; i < hi; ++i) {
    float acc = 0.0f;
    for (int j = 0; j < taps; ++j) {
      const int s = i - back + j;          // index among this step's tokens; negative: before the step
      float u = 0.0f;
      if (s >= 0) u = in[(size_t)(t0 + s) * ld_in + c];
      else if (pos0 + s >= 0) u = st[(size_t)(s + back) * C];
      acc = fmaf(wr[j], u, acc);
    }
    if (add_input) acc += in[(size_t)(t0 + i) * ld_in + c];
    if (act_silu) acc = acc / (1.0f + expf(-acc));
    out[(size_t)(t0 + i) * ldo + c] = from_f32<TO>(acc);
  }
  if (blockIdx.y == 0 && back > 0) {
    // the step's last inputs become the state; a step shorter than the state keeps the tail of the old one.
    // Row r is written after the rows it could still be read from (r + n > r), by the one thread that owns the channel.
    for (int r = 0; r < back; ++r) {
      const int s = n - back + r;
      st[(size_t)r * C] = s >= 0 ? in[(size_t)(t0 + s) * ld_in + c] : (pos0 + s >= 0 ? st[(size_t)(s + back) * C] : 0.0f);
    }
  }
}

extern "C" int hb_short_conv(int out_dtype, const float* in, int ld_in, const float* w, float* state, const int* seq_slot,
                             const int* seq_start, const int* seq_pos0, void* out, int ldo, int n_seqs, int max_q_len,
                             int channels, int taps, int add_input, int act_silu, void* stream) {
  HB_REQUIRE(n_seqs > 0 && max_q_len > 0 && channels > 0, "short_conv: sizes must be positive");
  HB_REQUIRE(taps >= 1 && taps - 1 <= SC_TOKENS, "short_conv: %d taps are outside the supported range 1..%d", taps, SC_TOKENS + 1);
  HB_REQUIRE(taps == 1 || state != nullptr, "short_conv: a convolution over more than one tap needs its state");
  HB_REQUIRE(n_seqs <= 65535 && ceil_div(max_q_len, SC_TOKENS) <= 65535, "short_conv: too many sequences or tokens per call");
  // tokens per CTA: fewer while the grid would leave SMs without several CTAs (a CTA's tokens are a serial loop)
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int span = SC_TOKENS;
  const int floor_span = taps - 1 > 8 ? taps - 1 : 8;
  while (span / 2 >= floor_span &&
         (long long)ceil_div(channels, SC_THREADS) * ceil_div(max_q_len, span) * n_seqs < 8LL * sms)
    span /= 2;
  dim3 grid(ceil_div(channels, SC_THREADS), ceil_div(max_q_len, span), n_seqs);
  if (out_dtype == HB_F32)
    hb_launch(short_conv_kernel<float>, grid, dim3(SC_THREADS), 0, (cudaStream_t)stream, in, ld_in, w, state, seq_slot, seq_start,
              seq_pos0, (float*)out, ldo, channels, taps, add_input, act_silu, span);
  else
    hb_launch(short_conv_kernel<bf16>, grid, dim3(SC_THREADS), 0, (cudaStream_t)stream, in, ld_in, w, state, seq_slot, seq_start,
              seq_pos0, (bf16*)out, ldo, channels, taps, add_input, act_silu, span);
  HB_CHECK_LAUNCH("short_conv");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// One CTA per token.  The CTA of a sequence's first token of the step reads the id the step before left in the slot
// and then leaves the step's last id there; no other CTA touches that int.
template <typename T>
__global__ void pair_embed_kernel(const T* __restrict__ table, const T* __restrict__ pair_table, const int* __restrict__ ids,
                                  const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                  const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int* __restrict__ last_id,
                                  float* __restrict__ out, int hidden, int vocab, int buckets, long long mul_prev,
                                  long long mul_cur, float scale) {
  __shared__ int prev_s;
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x;
  const int id = ids[t], b = tok_seq[t], p = tok_pos[t];
  const bool first = t == seq_start[b];
  if (threadIdx.x == 0) {
    int prev = -1;
    if (p > 0) prev = first ? last_id[seq_slot[b]] : ids[t - 1];
    prev_s = prev;
    if (first) last_id[seq_slot[b]] = ids[seq_start[b + 1] - 1];
  }
  __syncthreads();
  const int prev = prev_s;
  float* o = out + (size_t)t * hidden;
  if (id < 0 || id >= vocab) {  // the host validates ids; an invalid one yields zeros, never a stray read
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.0f;
    return;
  }
  long long row = buckets;
  if (prev >= 0) row = ((long long)prev * mul_prev + (long long)id * mul_cur) % (long long)buckets;
  if (row < 0) row += buckets;
  const T* er = table + (size_t)id * hidden;
  const T* pr = pair_table + (size_t)row * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_f32(er[i]) * scale + to_f32(pr[i]);
}

extern "C" int hb_pair_embed(int dtype, const void* table, const void* pair_table, const int* ids, const int* tok_seq,
                             const int* tok_pos, const int* seq_slot, const int* seq_start, int* last_id, float* out,
                             int n_tokens, int hidden, int vocab, int buckets, long long mul_prev, long long mul_cur,
                             float scale, void* stream) {
  HB_REQUIRE(n_tokens > 0 && hidden > 0 && vocab > 0 && buckets > 0, "pair_embed: sizes must be positive");
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == HB_F32)
    hb_launch(pair_embed_kernel<float>, dim3(n_tokens), dim3(threads), 0, (cudaStream_t)stream, (const float*)table,
              (const float*)pair_table, ids, tok_seq, tok_pos, seq_slot, seq_start, last_id, out, hidden, vocab, buckets, mul_prev,
              mul_cur, scale);
  else
    hb_launch(pair_embed_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, (cudaStream_t)stream, (const bf16*)table,
              (const bf16*)pair_table, ids, tok_seq, tok_pos, seq_slot, seq_start, last_id, out, hidden, vocab, buckets, mul_prev,
              mul_cur, scale);
  HB_CHECK_LAUNCH("pair_embed");
  return 0;
}
