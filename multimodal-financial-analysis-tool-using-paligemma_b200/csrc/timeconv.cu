// Short causal convolutions over time for ragged token batches, with the last inputs of every sequence kept as state.
//
// A convolution of `taps` taps over time on each channel reads, for the token at position p, the inputs of positions
// p - taps + 1 .. p of its sequence (zeros before the sequence's start).  In a step, the tokens of a sequence are
// consecutive rows at consecutive positions, so the input j positions back is row t - j when the sequence has that many
// rows before row t in this step, and otherwise comes from the sequence's state: the last taps - 1 inputs that earlier
// steps saw, fp32 [slots][taps - 1][channels], entry taps - 2 the most recent, all zero for a new sequence.  How many
// rows of its sequence precede a token is read off the token map (rows of one sequence carry the same slot).
//
// time_conv_residual_kernel : out = in + conv(in) on fp32 rows (the normalised residual stream), weights [C][taps]
//                             in the model dtype, the last column the current token's; fp32 sum, one rounding to the
//                             model dtype (the operand of the sublayer's projection).
// time_conv_state_kernel    : after the step's last reader of the state: per segment {slot, first row, tokens}, the
//                             state becomes the last taps - 1 entries of [old state ; the segment's inputs].  A
//                             thread owns a channel and writes the entries in ascending order, each from an older
//                             entry or from a row, so the update is in place.  Segments of 0 tokens are skipped.
//                             Its source is fp32 rows or model-dtype columns of a projection (the recurrent mixers'
//                             own convolutions keep their state the same way).
#include "common.cuh"

namespace pg {

template <typename T>
__global__ void __launch_bounds__(256)
time_conv_residual_kernel(T* __restrict__ out, const float* __restrict__ in, const T* __restrict__ w,
                          const float* __restrict__ state, const int32_t* __restrict__ tok_slot, int C, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, K = taps - 1;
  const int slot = tok_slot[t];
  int before = 0;                                  // rows of the same sequence right before this one, up to K
  while (before < K && t - before - 1 >= 0 && tok_slot[t - before - 1] == slot) ++before;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    const T* wc = w + (size_t)c * taps;
    const float cur = in[(size_t)t * C + c];
    float acc = cur * to_f<T>(wc[K]);
    for (int j = 1; j <= K; ++j) {
      const float v = j <= before ? in[(size_t)(t - j) * C + c]
                                  : state[((size_t)slot * K + (K - (j - before))) * C + c];
      acc = fmaf(v, to_f<T>(wc[K - j]), acc);
    }
    out[(size_t)t * C + c] = from_f<T>(cur + acc);
  }
}

template <typename TS>
__global__ void __launch_bounds__(256)
time_conv_state_kernel(float* __restrict__ state, const TS* __restrict__ src, int ld, int col0,
                       const int32_t* __restrict__ segs, int C, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int32_t* sg = segs + 3 * (size_t)blockIdx.x;
  const int slot = sg[0], row0 = sg[1], n = sg[2], K = taps - 1;
  if (n <= 0) return;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float* st = state + (size_t)slot * K * C + c;
    for (int i = 0; i < K; ++i) {                  // entry i of the new state = entry n + i of [old state ; rows]
      const int idx = n + i;
      st[(size_t)i * C] = idx < K ? st[(size_t)idx * C] : to_f<TS>(src[(size_t)(row0 + idx - K) * ld + col0 + c]);
    }
  }
}

}  // namespace pg

using namespace pg;

extern "C" int pg_time_conv_residual(void* out, const float* in, const void* w, const float* state,
                                     const int32_t* tok_slot, int n_tokens, int C, int taps, int dtype, void* stream) {
  if (n_tokens <= 0) return PG_OK;
  PG_REQUIRE(out && in && w && tok_slot && C > 0 && taps >= 1 && (taps == 1 || state), "time_conv_residual: bad arguments");
  PG_DISPATCH_DTYPE(dtype, T, {
    return launch_pdl("time_conv_residual", time_conv_residual_kernel<T>, dim3(n_tokens, cdiv(C, 1024)), dim3(256), 0,
                      (cudaStream_t)stream, (T*)out, in, (const T*)w, state, tok_slot, C, taps);
  });
  return PG_OK;
}

extern "C" int pg_time_conv_state(float* state, const void* src, int ld, int col0, int src_f32, const int32_t* segs,
                                  int n_segs, int C, int taps, int dtype, void* stream) {
  if (n_segs <= 0 || taps <= 1) return PG_OK;
  PG_REQUIRE(state && src && segs && C > 0 && ld >= C, "time_conv_state: bad arguments");
  const dim3 grid(n_segs, cdiv(C, 256));
  if (src_f32)
    return launch_pdl("time_conv_state", time_conv_state_kernel<float>, grid, dim3(256), 0, (cudaStream_t)stream, state,
                      (const float*)src, ld, col0, segs, C, taps);
  PG_DISPATCH_DTYPE(dtype, T, {
    return launch_pdl("time_conv_state", time_conv_state_kernel<T>, grid, dim3(256), 0, (cudaStream_t)stream, state,
                      (const T*)src, ld, col0, segs, C, taps);
  });
  return PG_OK;
}
