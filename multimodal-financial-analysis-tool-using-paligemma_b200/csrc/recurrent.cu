// Recurrent mixers for ragged token batches: the generalised delta rule with a per-channel decay, and lightning
// attention (linear attention with a constant decay per head; described at its kernel below).
//
// Per head, with a state S [dim x dim] (key channel i, value column j) kept in fp32 per sequence slot:
//     u   = k / sqrt(sum(k^2) + key_eps)
//     S  <- diag(w) S - (a * u) (u^T S) + k v^T          (both first terms read the old S)
//     o   = S^T r
// Everything that enters the recurrence besides the projections themselves is fp32: the decay w, the removal rate a,
// the unit key u, the state and the output.
//
// delta_prep_kernel   (CTA per 8 tokens) : w = exp(-decay_scale * sigmoid(W2 tanh(inner) + w0)) with the W2 product in
//                                         fp32 (a thread owns a channel and walks its W2 row once for the CTA's
//                                         tokens), a = sigmoid(a_pre + a_bias), u; writes one packed fp32 record
//                                         [r | k | w | u | a*u | v] x dp (dp = dim rounded up to 4) per (token, head),
//                                         so that the recurrence streams ONE contiguous block per token and head.
// delta_rule_kernel   (CTA per (sequence segment, head)): the state lives in registers, a thread owning a quarter of
//                                         one value column; the u^T S and S^T r products are per-thread dot products
//                                         with vectors read from shared memory plus two shuffle steps, so the tokens
//                                         of a segment need no block-wide exchange.  The records of the next
//                                         tokens arrive by cp.async into the other half of a double buffer while
//                                         the current ones are consumed.  The state is loaded from / stored to the
//                                         slot's state once per launch, which makes a prompt portion and a single
//                                         decoded token the same case.
// headnorm_gate_kernel (warp per (token, head)): o / rms(o) per head, times a weight, times sigmoid(gate), times a
//                                         constant, rounded to the model dtype as the output projection's operand.
#include "common.cuh"

namespace pg {

__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }

constexpr int PREP_TOK = 8;     // tokens per CTA of the prep kernel
constexpr int REC_VECS = 6;     // r, k, w, u, a*u, v
enum { REC_R = 0, REC_K = 1, REC_W = 2, REC_U = 3, REC_AU = 4, REC_V = 5 };

template <typename T>
__global__ void __launch_bounds__(256)
delta_prep_kernel(float* __restrict__ rec, const T* __restrict__ proj, int ld, int r_col0, int k_col0, int v_col0,
                  int a_col0, int lora_col0, int lora, const T* __restrict__ w2, const T* __restrict__ w0,
                  const T* __restrict__ a_bias, int n_tokens, int heads, int dim, int dp, float decay_scale,
                  float key_eps) {
  extern __shared__ float sm[];           // [PREP_TOK][lora] tanh of the decay's inner projection | [PREP_TOK][heads] sum k^2
  float* lo = sm;
  float* ksq = sm + PREP_TOK * lora;
  pdl_launch_dependents();
  pdl_wait();
  const int t0 = blockIdx.x * PREP_TOK, nt = min(PREP_TOK, n_tokens - t0), nd = heads * dim;
  for (int idx = threadIdx.x; idx < PREP_TOK * lora; idx += blockDim.x) {
    const int tt = idx / lora, j = idx % lora;
    lo[idx] = tt < nt ? tanhf(to_f<T>(proj[(size_t)(t0 + tt) * ld + lora_col0 + j])) : 0.f;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int item = warp; item < nt * heads; item += warps) {
    const int tt = item / heads, h = item % heads;
    const T* kr = proj + (size_t)(t0 + tt) * ld + k_col0 + h * dim;
    float s = 0.f;
    for (int c = lane; c < dim; c += 32) { const float v = to_f<T>(kr[c]); s += v * v; }
    s = warp_sum(s);
    if (lane == 0) ksq[tt * heads + h] = s;
  }
  __syncthreads();
  constexpr int V = Vec<T>::N;
  const bool vec = (lora % V) == 0 && (reinterpret_cast<uintptr_t>(w2) & 15) == 0;
  // blockIdx.y cuts the channels into slices of c_per (a handful of tokens: more CTAs than token groups)
  const int c_per = (nd + gridDim.y - 1) / gridDim.y, c_end = min(nd, (int)(blockIdx.y + 1) * c_per);
  for (int c = blockIdx.y * c_per + threadIdx.x; c < c_end; c += blockDim.x) {
    float z[PREP_TOK];
    const float z0 = to_f<T>(w0[c]);
#pragma unroll
    for (int tt = 0; tt < PREP_TOK; ++tt) z[tt] = z0;
    const T* wr = w2 + (size_t)c * lora;
    if (vec) {
      for (int j = 0; j < lora; j += V) {
        float f[V];
        unpack<T>(*reinterpret_cast<const uint4*>(wr + j), f);
#pragma unroll
        for (int tt = 0; tt < PREP_TOK; ++tt)
#pragma unroll
          for (int i = 0; i < V; ++i) z[tt] = fmaf(f[i], lo[tt * lora + j + i], z[tt]);
      }
    } else {
      for (int j = 0; j < lora; ++j) {
        const float f = to_f<T>(wr[j]);
#pragma unroll
        for (int tt = 0; tt < PREP_TOK; ++tt) z[tt] = fmaf(f, lo[tt * lora + j], z[tt]);
      }
    }
    const int h = c / dim, i = c % dim;
    const float ab = a_bias ? to_f<T>(a_bias[c]) : 0.f;
#pragma unroll
    for (int tt = 0; tt < PREP_TOK; ++tt) {
      if (tt >= nt) break;
      const T* row = proj + (size_t)(t0 + tt) * ld;
      const float k = to_f<T>(row[k_col0 + c]);
      const float u = k / sqrtf(ksq[tt * heads + h] + key_eps);
      float* o = rec + (((size_t)(t0 + tt) * heads + h) * REC_VECS) * dp + i;
      o[REC_R * dp] = to_f<T>(row[r_col0 + c]);
      o[REC_K * dp] = k;
      o[REC_W * dp] = expf(-decay_scale * sigmoid_f(z[tt]));
      o[REC_U * dp] = u;
      o[REC_AU * dp] = sigmoid_f(to_f<T>(row[a_col0 + c]) + ab) * u;
      o[REC_V * dp] = to_f<T>(row[v_col0 + c]);
    }
  }
  // the padding columns of every record are zero, so the recurrence can run whole 4-wide groups
  const int pad = dp - dim;
  if (pad && blockIdx.y == 0)
    for (int idx = threadIdx.x; idx < nt * heads * REC_VECS * pad; idx += blockDim.x) {
      const int i = dim + idx % pad, which = idx / pad;
      rec[((size_t)t0 * heads * REC_VECS + which) * dp + i] = 0.f;
    }
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// segs: [n_segs][3] = {state slot, first token row, tokens}; the tokens of a segment are consecutive rows of one
// sequence in position order.  A segment with 0 tokens is skipped (the list is padded to a fixed length so that a
// captured launch stays valid).  Shared memory: two buffers of CH records.
template <int DMAX, int CH>
__global__ void __launch_bounds__(DMAX * 4)
delta_rule_kernel(float* __restrict__ out, float* __restrict__ state, const float* __restrict__ rec,
                  const int32_t* __restrict__ segs, int heads, int dim, int dp) {
  // thread = (value column j, row group rg): of column j it keeps the rows 4 (m RG + rg) + e (m < NG, e < 4) in
  // registers, i.e. every RG-th group of four rows, so that the four row groups of a column (adjacent lanes) read four
  // consecutive 16-byte pieces of a vector (no bank conflict) and the two column sums of a token are two shuffle
  // steps each.  Vectors sit in shared memory with stride DMAX and zeros behind dim: no bound checks in the token loop.
  constexpr int RG = 4, NG = DMAX / (4 * RG);
  extern __shared__ __align__(16) float sh[];       // [2][CH][REC_VECS][DMAX]
  pdl_launch_dependents();
  pdl_wait();
  const int32_t* sg = segs + 3 * (size_t)blockIdx.x;
  const int slot = sg[0], row0 = sg[1], n = sg[2];
  if (n <= 0) return;
  const int h = blockIdx.y, j = blockIdx.z * (blockDim.x / RG) + threadIdx.x / RG, rg = threadIdx.x % RG, nd = heads * dim;
  const bool live = j < dim;
  constexpr int RSZ = REC_VECS * DMAX;              // floats of one record in shared memory
  if (dp < DMAX)
    for (int idx = threadIdx.x; idx < 2 * CH * RSZ; idx += blockDim.x)
      if (idx % DMAX >= dp) sh[idx] = 0.f;
  float S[NG * 4];
  float* st = state + ((size_t)slot * heads + h) * dim * dim;
#pragma unroll
  for (int m = 0; m < NG; ++m)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = 4 * (m * RG + rg) + e;
      S[m * 4 + e] = (live && i < dim) ? st[(size_t)i * dim + j] : 0.f;
    }
  const int vp = dp / 4, pieces = REC_VECS * vp;    // 16-byte pieces of one vector / one record
  auto fetch = [&](int t0, int buf) {               // records of tokens [t0, t0 + CH) of this head -> buffer buf
    const int nt = min(CH, n - t0);
    for (int idx = threadIdx.x; idx < nt * pieces; idx += blockDim.x) {
      const int tt = idx / pieces, rem = idx % pieces, v = rem / vp, pc = rem % vp;
      cp_async16(sh + ((size_t)buf * CH + tt) * RSZ + v * DMAX + pc * 4,
                 rec + (((size_t)row0 + t0 + tt) * heads + h) * (size_t)(REC_VECS * dp) + v * dp + pc * 4);
    }
    cp_async_commit();
  };
  fetch(0, 0);
  int buf = 0;
  for (int t0 = 0; t0 < n; t0 += CH, buf ^= 1) {
    const int nt = min(CH, n - t0);
    if (t0 + CH < n) { fetch(t0 + CH, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
#pragma unroll 2
    for (int tt = 0; tt < nt; ++tt) {
      const float* r = sh + ((size_t)buf * CH + tt) * RSZ + 4 * rg;
      const float vj = r[REC_V * DMAX + j - 4 * rg];
      float4 u4[NG], w4[NG], a4[NG], k4[NG], r4[NG];
#pragma unroll
      for (int m = 0; m < NG; ++m) {
        u4[m] = *reinterpret_cast<const float4*>(r + REC_U * DMAX + 16 * m);
        w4[m] = *reinterpret_cast<const float4*>(r + REC_W * DMAX + 16 * m);
        a4[m] = *reinterpret_cast<const float4*>(r + REC_AU * DMAX + 16 * m);
        k4[m] = *reinterpret_cast<const float4*>(r + REC_K * DMAX + 16 * m);
        r4[m] = *reinterpret_cast<const float4*>(r + REC_R * DMAX + 16 * m);
      }
      float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;            // this thread's part of u^T S for column j
#pragma unroll
      for (int m = 0; m < NG; ++m) {
        d0 = fmaf(u4[m].x, S[4 * m], d0); d1 = fmaf(u4[m].y, S[4 * m + 1], d1);
        d2 = fmaf(u4[m].z, S[4 * m + 2], d2); d3 = fmaf(u4[m].w, S[4 * m + 3], d3);
      }
      float us = (d0 + d1) + (d2 + d3);
      us += __shfl_xor_sync(0xffffffffu, us, 1);
      us += __shfl_xor_sync(0xffffffffu, us, 2);
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int m = 0; m < NG; ++m) {
        S[4 * m] = fmaf(k4[m].x, vj, fmaf(-a4[m].x, us, w4[m].x * S[4 * m]));
        S[4 * m + 1] = fmaf(k4[m].y, vj, fmaf(-a4[m].y, us, w4[m].y * S[4 * m + 1]));
        S[4 * m + 2] = fmaf(k4[m].z, vj, fmaf(-a4[m].z, us, w4[m].z * S[4 * m + 2]));
        S[4 * m + 3] = fmaf(k4[m].w, vj, fmaf(-a4[m].w, us, w4[m].w * S[4 * m + 3]));
        o0 = fmaf(r4[m].x, S[4 * m], o0); o1 = fmaf(r4[m].y, S[4 * m + 1], o1);
        o2 = fmaf(r4[m].z, S[4 * m + 2], o2); o3 = fmaf(r4[m].w, S[4 * m + 3], o3);
      }
      float o = (o0 + o1) + (o2 + o3);
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      if (live && rg == 0) out[((size_t)row0 + t0 + tt) * nd + h * dim + j] = o;
    }
    __syncthreads();                                // every thread is done with this buffer before it is refilled
  }
  if (live) {
#pragma unroll
    for (int m = 0; m < NG; ++m)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = 4 * (m * RG + rg) + e;
        if (i < dim) st[(size_t)i * dim + j] = S[m * 4 + e];
      }
  }
}

template <typename T>
__global__ void headnorm_gate_kernel(T* __restrict__ out, int ld_out, const float* __restrict__ o, const T* __restrict__ w,
                                     const T* __restrict__ gate, int ld_gate, int n_tokens, int heads, int dim, float eps,
                                     float out_scale, int pairs) {
  pdl_launch_dependents();
  pdl_wait();
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= (long long)n_tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item % heads);
  const float* orow = o + ((size_t)t * heads + h) * dim;
  float ss = 0.f;
  if (pairs) {                                     // two columns per lane and access (even sizes, aligned rows)
    for (int c = 2 * lane; c < dim; c += 64) { const float2 v = *reinterpret_cast<const float2*>(orow + c); ss += v.x * v.x + v.y * v.y; }
    ss = warp_sum(ss);
    const float inv = out_scale / sqrtf(ss / (float)dim + eps);
    for (int c = 2 * lane; c < dim; c += 64) {
      const float2 v = *reinterpret_cast<const float2*>(orow + c);
      float a = v.x * inv, b = v.y * inv;
      if (w) { a *= to_f<T>(w[h * dim + c]); b *= to_f<T>(w[h * dim + c + 1]); }
      if (gate) {
        const T* gp = gate + (size_t)t * ld_gate + h * dim + c;
        a *= sigmoid_f(to_f<T>(gp[0])); b *= sigmoid_f(to_f<T>(gp[1]));
      }
      T* op = out + (size_t)t * ld_out + h * dim + c;
      if constexpr (sizeof(T) == 2) {
        T two[2] = {from_f<T>(a), from_f<T>(b)};
        *reinterpret_cast<uint32_t*>(op) = *reinterpret_cast<const uint32_t*>(two);
      } else {
        op[0] = from_f<T>(a); op[1] = from_f<T>(b);
      }
    }
    return;
  }
  for (int c = lane; c < dim; c += 32) ss += orow[c] * orow[c];
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)dim + eps);
  for (int c = lane; c < dim; c += 32) {
    float v = orow[c] * inv;
    if (w) v *= to_f<T>(w[h * dim + c]);
    if (gate) v *= sigmoid_f(to_f<T>(gate[(size_t)t * ld_gate + h * dim + c]));
    out[(size_t)t * ld_out + h * dim + c] = from_f<T>(v * out_scale);
  }
}

// ------------------------------------------------------------------ lightning attention: linear attention with a constant decay per head
// Per head, with a state S [dim x vdim] (key channel i, value column j) kept in fp32 per sequence slot:
//     q = silu(q_pre), k = silu(k_pre), v = silu(v_pre)          (pre-activations: the fused projection, model dtype)
//     S <- decay_h S + k v^T,        o = S^T q
// lightning_prep_kernel  (elementwise)  the activations in fp32, one packed record [q | k | v] per (token, head) with
//                                       q, k padded to dp = dim rounded up to 4 floats and v to vp likewise (zeros).
// lightning_kernel       (CTA per (sequence segment, head, slice of VT value columns)): a thread owns a quarter of
//                                       the rows of one value column (the layout of the delta-rule kernel above: rows
//                                       4 (m RG + rg) + e), so a token costs one fused multiply-add per state element
//                                       for the update, one for the output, and two shuffle steps.  The records of
//                                       the next CH tokens arrive by cp.async into the other half of a double buffer.
//                                       The state is read from and written back to the slot once per launch, which
//                                       makes a prompt portion and a single decoded token the same case and the
//                                       result independent of where the sequence was cut.
template <typename T>
__global__ void lightning_prep_kernel(float* __restrict__ rec, const T* __restrict__ proj, int ld, int q_col0, int k_col0,
                                      int v_col0, long long n_tokens, int heads, int dim, int vdim, int dp, int vp) {
  pdl_launch_dependents();
  pdl_wait();
  const int rs = 2 * dp + vp;                       // floats of one record
  // blockIdx.x: token; the CTA's threads walk the token's heads x record columns
  const long long t = blockIdx.x;
  const T* row = proj + t * ld;
  float* out = rec + t * heads * rs;
  for (int i = threadIdx.x; i < heads * rs; i += blockDim.x) {
    const int h = i / rs, c = i - h * rs;
    int col = -1;
    if (c < dp) { if (c < dim) col = q_col0 + h * dim + c; }
    else if (c < 2 * dp) { if (c - dp < dim) col = k_col0 + h * dim + c - dp; }
    else if (c - 2 * dp < vdim) col = v_col0 + h * vdim + c - 2 * dp;
    float a = 0.f;
    if (col >= 0) {
      a = to_f<T>(row[col]);
      a = a * sigmoid_f(a);
    }
    out[i] = a;
  }
}

//                                       TD (decay per token): the record carries four more floats [decay, 0, 0, 0] after
//                                       the values and the decay of a token comes from there instead of decay[h];
//                                       skip (may be NULL): skip[h] * v is added to the output (the state-space
//                                       mixer's direct term, with v its unscaled input).
template <int DMAX, int RG, int CH, bool TD>
__global__ void __launch_bounds__(256)
lightning_kernel(float* __restrict__ out, float* __restrict__ state, const float* __restrict__ rec,
                 const float* __restrict__ decay, const float* __restrict__ skip, const int32_t* __restrict__ segs,
                 int heads, int dim, int vdim, int dp, int vp) {
  constexpr int NG = DMAX / (4 * RG);               // groups of four rows per thread (RG lanes share a value column)
  extern __shared__ __align__(16) float sh[];       // [2][CH][q DMAX | k DMAX | v VT]
  pdl_launch_dependents();
  pdl_wait();
  const int32_t* sg = segs + 3 * (size_t)blockIdx.x;
  const int slot = sg[0], row0 = sg[1], n = sg[2];
  if (n <= 0) return;
  constexpr int XP = TD ? 4 : 0;
  const int VT = blockDim.x / RG, RSZ = 2 * DMAX + VT + XP, rs = 2 * dp + vp + XP;
  const int h = blockIdx.y, j0 = blockIdx.z * VT, jl = threadIdx.x / RG, j = j0 + jl, rg = threadIdx.x % RG;
  const bool live = j < vdim;
  const float lam_h = TD ? 0.f : decay[h], skip_h = skip ? skip[h] : 0.f;
  for (int idx = threadIdx.x; idx < 2 * CH * RSZ; idx += blockDim.x) sh[idx] = 0.f;   // padding the copies never write
  float S[NG * 4];
  float* st = state + ((size_t)slot * heads + h) * dim * vdim;
#pragma unroll
  for (int m = 0; m < NG; ++m)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = 4 * (m * RG + rg) + e;
      S[m * 4 + e] = (live && i < dim) ? st[(size_t)i * vdim + j] : 0.f;
    }
  __syncthreads();
  const int qk_pieces = dp / 4, v_pieces = min(VT, vp - j0) / 4, pieces = 2 * qk_pieces + v_pieces + (TD ? 1 : 0);
  auto fetch = [&](int t0, int buf) {               // records of tokens [t0, t0 + CH) of this head -> buffer buf
    const int nt = min(CH, n - t0);
    for (int idx = threadIdx.x; idx < nt * pieces; idx += blockDim.x) {
      const int tt = idx / pieces, pc = idx % pieces;
      const float* src = rec + (((size_t)row0 + t0 + tt) * heads + h) * (size_t)rs;
      float* dst = sh + ((size_t)buf * CH + tt) * RSZ;
      if (pc < qk_pieces) cp_async16(dst + pc * 4, src + pc * 4);
      else if (pc < 2 * qk_pieces) cp_async16(dst + DMAX + (pc - qk_pieces) * 4, src + dp + (pc - qk_pieces) * 4);
      else if (pc < 2 * qk_pieces + v_pieces) cp_async16(dst + 2 * DMAX + (pc - 2 * qk_pieces) * 4, src + 2 * dp + j0 + (pc - 2 * qk_pieces) * 4);
      else cp_async16(dst + 2 * DMAX + VT, src + 2 * dp + vp);
    }
    cp_async_commit();
  };
  fetch(0, 0);
  int buf = 0;
  for (int t0 = 0; t0 < n; t0 += CH, buf ^= 1) {
    const int nt = min(CH, n - t0);
    if (t0 + CH < n) { fetch(t0 + CH, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
#pragma unroll 2
    for (int tt = 0; tt < nt; ++tt) {
      const float* r = sh + ((size_t)buf * CH + tt) * RSZ;
      const float vj = r[2 * DMAX + jl];
      const float lam = TD ? r[2 * DMAX + VT] : lam_h;
      const float* qr = r + 4 * rg;
      const float* kr = r + DMAX + 4 * rg;
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int m = 0; m < NG; ++m) {
        const float4 k4 = *reinterpret_cast<const float4*>(kr + 4 * RG * m);
        const float4 q4 = *reinterpret_cast<const float4*>(qr + 4 * RG * m);
        S[4 * m] = fmaf(k4.x, vj, lam * S[4 * m]);
        S[4 * m + 1] = fmaf(k4.y, vj, lam * S[4 * m + 1]);
        S[4 * m + 2] = fmaf(k4.z, vj, lam * S[4 * m + 2]);
        S[4 * m + 3] = fmaf(k4.w, vj, lam * S[4 * m + 3]);
        o0 = fmaf(q4.x, S[4 * m], o0); o1 = fmaf(q4.y, S[4 * m + 1], o1);
        o2 = fmaf(q4.z, S[4 * m + 2], o2); o3 = fmaf(q4.w, S[4 * m + 3], o3);
      }
      float o = (o0 + o1) + (o2 + o3);
#pragma unroll
      for (int sh_ = 1; sh_ < RG; sh_ <<= 1) o += __shfl_xor_sync(0xffffffffu, o, sh_);
      if (live && rg == 0) out[((size_t)row0 + t0 + tt) * heads * vdim + h * vdim + j] = fmaf(skip_h, vj, o);
    }
    __syncthreads();                                // every thread is done with this buffer before it is refilled
  }
  if (live) {
#pragma unroll
    for (int m = 0; m < NG; ++m)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = 4 * (m * RG + rg) + e;
        if (i < dim) st[(size_t)i * vdim + j] = S[m * 4 + e];
      }
  }
}

template <int DMAX, int RG, int CH>
static int launch_lightning(float* out, float* state, const float* rec, const float* decay, const float* skip, bool td,
                            const int32_t* segs, int n_segs, int heads, int dim, int vdim, cudaStream_t st) {
  const int dp = (dim + 3) / 4 * 4, vp = (vdim + 3) / 4 * 4;
  // value columns per CTA: as many as 256 threads hold for prompt-sized work (few fat CTAs, about one per SM, beat
  // many thin ones: 0.75 against 0.87 ms at 4 x 2048 tokens, 8 heads of 128), fewer while the CTAs do not fill the SMs
  int vt = 256 / RG;
  while (vt > 8 && (vt / 2 >= vdim || (long long)n_segs * heads * cdiv(vdim, vt) < 100)) vt /= 2;
  static const int vt_env = env_int("PG_LIGHTNING_VT", 0);
  if (vt_env >= 8 && vt_env <= 256 / RG && (vt_env & (vt_env - 1)) == 0) vt = vt_env;
  const size_t smem = sizeof(float) * 2 * CH * (2 * DMAX + vt + (td ? 4 : 0));
  // An ordinary launch, not a programmatic dependent one: CTAs that become resident while the preceding kernel still
  // fills the machine are placed on the few SMs with room, and a recurrence of a few hundred long-lived CTAs then runs
  // on a fraction of the GPU (measured at 4 x 2048 tokens, 8 heads of 128: 2.06 ms against 0.88 ms).
  if (td)
    lightning_kernel<DMAX, RG, CH, true><<<dim3(n_segs, heads, cdiv(vdim, vt)), dim3(vt * RG), smem, st>>>(
        out, state, rec, decay, skip, segs, heads, dim, vdim, dp, vp);
  else
    lightning_kernel<DMAX, RG, CH, false><<<dim3(n_segs, heads, cdiv(vdim, vt)), dim3(vt * RG), smem, st>>>(
        out, state, rec, decay, skip, segs, heads, dim, vdim, dp, vp);
  return check_launch("lightning");
}

template <int DMAX, int CH>
static int launch_delta(float* out, float* state, const float* rec, const int32_t* segs, int n_segs, int heads, int dim,
                        cudaStream_t st) {
  const int dp = (dim + 3) / 4 * 4;
  const size_t smem = sizeof(float) * 2 * CH * REC_VECS * DMAX;
  // few (segment, head) pairs: the value columns of a head are cut over `cut` CTAs (each fetches the head's records)
  static const int cut_env = env_int("PG_DELTA_COLUMN_CUT", 0);
  int cut = 1;
  if (DMAX >= 16 && (long long)n_segs * heads * 2 <= 160) cut = 2;   // measured: 0.95 -> 0.68 ms at 64 pairs, slower from 128 on
  if (cut_env > 0 && DMAX / cut_env >= 8) cut = cut_env;
  return launch_pdl("delta_rule", delta_rule_kernel<DMAX, CH>, dim3(n_segs, heads, cut), dim3(DMAX * 4 / cut), smem, st, out, state,
                    rec, segs, heads, dim, dp);
}

}  // namespace pg

using namespace pg;

extern "C" long long pg_delta_record_floats(int n_tokens, int heads, int dim) {
  return (long long)n_tokens * heads * REC_VECS * ((dim + 3) / 4 * 4);
}

extern "C" int pg_delta_prep(float* rec, const void* proj, int ld, int r_col0, int k_col0, int v_col0, int a_col0,
                             int lora_col0, int lora, const void* w2, const void* w0, const void* a_bias, int n_tokens,
                             int heads, int dim, float decay_scale, float key_eps, int dtype, void* stream) {
  if (n_tokens <= 0) return PG_OK;
  PG_REQUIRE(rec && proj && w2 && w0 && lora > 0 && heads > 0 && dim > 0, "delta_prep: bad arguments");
  const size_t smem = sizeof(float) * PREP_TOK * ((size_t)lora + heads);
  PG_DISPATCH_DTYPE(dtype, T, {
    const int threads = heads * dim >= 256 ? 256 : 128;
    const int slices = n_tokens <= 64 ? cdiv(heads * dim, threads) : 1;
    return launch_pdl("delta_prep", delta_prep_kernel<T>, dim3(cdiv(n_tokens, PREP_TOK), slices), dim3(threads),
                      smem, (cudaStream_t)stream, rec, (const T*)proj, ld, r_col0, k_col0, v_col0, a_col0, lora_col0, lora,
                      (const T*)w2, (const T*)w0, (const T*)a_bias, n_tokens, heads, dim, (dim + 3) / 4 * 4, decay_scale,
                      key_eps);
  });
  return PG_OK;
}

extern "C" int pg_delta_rule(float* out, float* state, const float* rec, const int32_t* segs, int n_segs, int heads,
                             int dim, void* stream) {
  if (n_segs <= 0) return PG_OK;
  PG_REQUIRE(out && state && rec && segs, "delta_rule: bad arguments");
  PG_REQUIRE(dim > 0 && dim <= 256, "delta_rule: head size %d (1..256)", dim);
  cudaStream_t st = (cudaStream_t)stream;
  if (dim <= 32) return launch_delta<32, 8>(out, state, rec, segs, n_segs, heads, dim, st);
  if (dim <= 64) return launch_delta<64, 8>(out, state, rec, segs, n_segs, heads, dim, st);
  if (dim <= 128) return launch_delta<128, 4>(out, state, rec, segs, n_segs, heads, dim, st);
  return launch_delta<256, 2>(out, state, rec, segs, n_segs, heads, dim, st);
}

extern "C" int pg_headnorm_gate(void* out, int ld_out, const float* o, const void* w, const void* gate, int ld_gate,
                                int n_tokens, int heads, int dim, float eps, float out_scale, int dtype, void* stream) {
  if (n_tokens <= 0) return PG_OK;
  PG_REQUIRE(out && o && heads > 0 && dim > 0, "headnorm_gate: bad arguments");
  const int warps = 8;
  const int pairs = (dim % 2 == 0 && ld_out % 2 == 0 && ld_gate % 2 == 0 && ((uintptr_t)out % 4) == 0 &&
                     ((uintptr_t)o % 8) == 0) ? 1 : 0;
  PG_DISPATCH_DTYPE(dtype, T, {
    return launch_pdl("headnorm_gate", headnorm_gate_kernel<T>, dim3(cdiv((long long)n_tokens * heads, warps)),
                      dim3(warps * 32), 0, (cudaStream_t)stream, (T*)out, ld_out, o, (const T*)w, (const T*)gate, ld_gate,
                      n_tokens, heads, dim, eps, out_scale, pairs);
  });
  return PG_OK;
}

extern "C" long long pg_lightning_record_floats(int n_tokens, int heads, int dim, int vdim) {
  return (long long)n_tokens * heads * (2 * ((dim + 3) / 4 * 4) + (vdim + 3) / 4 * 4);
}

extern "C" int pg_lightning_prep(float* rec, const void* proj, int ld, int q_col0, int k_col0, int v_col0, int n_tokens,
                                 int heads, int dim, int vdim, int dtype, void* stream) {
  if (n_tokens <= 0) return PG_OK;
  PG_REQUIRE(rec && proj && heads > 0 && dim > 0 && vdim > 0, "lightning_prep: bad arguments");
  const int dp = (dim + 3) / 4 * 4, vp = (vdim + 3) / 4 * 4;
  PG_DISPATCH_DTYPE(dtype, T, {
    return launch_pdl("lightning_prep", lightning_prep_kernel<T>, dim3(n_tokens), dim3(256), 0, (cudaStream_t)stream, rec,
                      (const T*)proj, ld, q_col0, k_col0, v_col0, (long long)n_tokens, heads, dim, vdim, dp, vp);
  });
  return PG_OK;
}

extern "C" int pg_lightning_attention(float* out, float* state, const float* rec, const float* decay, const int32_t* segs,
                                      int n_segs, int heads, int dim, int vdim, void* stream) {
  return pg_lightning_attention_ex(out, state, rec, decay, nullptr, segs, n_segs, heads, dim, vdim, stream);
}

extern "C" int pg_lightning_attention_ex(float* out, float* state, const float* rec, const float* decay, const float* skip,
                                         const int32_t* segs, int n_segs, int heads, int dim, int vdim, void* stream) {
  if (n_segs <= 0) return PG_OK;
  const bool td = decay == nullptr;                 // no constant decay: the records carry one per token
  PG_REQUIRE(out && state && rec && segs, "lightning_attention: bad arguments");
  PG_REQUIRE(dim > 0 && dim <= 256 && vdim > 0, "lightning_attention: key size %d (1..256), value size %d", dim, vdim);
  cudaStream_t st = (cudaStream_t)stream;
  // lanes per value column: a thread keeps DMAX / RG state elements, and a token is that many fused multiply-adds
  // twice plus log2(RG) shuffle steps on the critical path of the recurrence
  if (dim <= 32) return launch_lightning<32, 4, 16>(out, state, rec, decay, skip, td, segs, n_segs, heads, dim, vdim, st);
  // tokens per buffer: the next buffer's records must be on their way for longer than a DRAM round trip while this
  // one is consumed (16 tokens of 64..128 key channels; 8 left the recurrence waiting on every refill)
  static const int deep = env_int("PG_LIGHTNING_DEEP", 1);
  if (dim <= 64)
    return deep ? launch_lightning<64, 8, 16>(out, state, rec, decay, skip, td, segs, n_segs, heads, dim, vdim, st)
                : launch_lightning<64, 8, 8>(out, state, rec, decay, skip, td, segs, n_segs, heads, dim, vdim, st);
  if (dim <= 128)
    return deep ? launch_lightning<128, 8, 16>(out, state, rec, decay, skip, td, segs, n_segs, heads, dim, vdim, st)
                : launch_lightning<128, 8, 8>(out, state, rec, decay, skip, td, segs, n_segs, heads, dim, vdim, st);
  return launch_lightning<256, 16, 4>(out, state, rec, decay, skip, td, segs, n_segs, heads, dim, vdim, st);
}
