// Causal attention over the paged cache for ragged token batches: sliding window, per-head distance bias,
// grouped key/value heads, separate key and value widths, optional sigmoid output gate.
//
// Token t of the step sits at position p = tok_pos[t] of the sequence whose pages are row tok_slot[t] of the page
// table; its keys are the positions j with 0 <= p - j < window (window <= 0: all j <= p) of that sequence, which the
// append kernel has written before this launch (the step's own tokens included), so a prompt portion and a single
// decoded token are the same case.  score = (q . k_j) * scale - slope[h] * (p - j); fp32 scores, softmax weights and
// accumulation; out = softmax(score) V, times sigmoid(gate) when a gate is given, rounded once to the model dtype.
//
// Extensions (pg_attention_ragged_ex): keep_first > 0 keeps the first keep_first positions of the sequence visible
// behind the window (they keep their true positions); the visible keys of a token are then the virtual list
// [0, min(keep_first, lo)) ++ [lo, p], which every kernel below walks through one index map.  weights == 1 replaces
// the softmax by unnormalised weights sigmoid(score + head_bias[h]).  The gate is either one value per output column
// (gate_per_head == 0) or one per (token, head); the result is multiplied by out_scale before the single rounding.
// pg_attention_ragged_sink adds: sink[h], a per-head logit without key or value whose exp joins the softmax
// denominator once (after all partial sums are merged), and explicit row strides of the key and the value pool, so
// that the value rows may be a prefix of the key rows of ONE pool (latent attention: key [c | k_rot], value c).
//
// attention_ragged_kernel: one warp per (token, head).  32 keys per iteration, one key per lane for the dot
// product (the query row lives in shared memory as fp32), running (max, sum) rescaling, then the lanes switch to the
// value columns and walk the 32 keys with the weights broadcast by shuffles.  Warps of a CTA are the heads of the
// same token and its neighbours, so the key / value rows they share are served by L1.
//
// attention_ragged_split_kernel: decode-sized batches (a handful of tokens): one CTA per (token, key/value head, key
// slice) serves all query heads of the group (or a chunk of 8 / 4 / 2 of them, when the group is larger or the value
// rows are wide) from ONE read of every key and value row; the keys are split over key
// slices (CTAs) and over the warps of a CTA; the partial (max, sum, acc) triples are merged through shared memory
// and, across slices, through a caller-owned fp32 workspace by attention_ragged_merge_kernel, always in a fixed
// order.  A lane owns ceil(vdim / 32) contiguous value columns, fetched with one vector load per key.
#include "common.cuh"

namespace pg {

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ qs, const T* __restrict__ kp, int dim) {
  constexpr int V = Vec<T>::N;
  float acc = 0.f;
  if ((dim % V) == 0 && (reinterpret_cast<uintptr_t>(kp) & 15) == 0) {
    int c = 0;
    float a1 = 0.f, a2 = 0.f, a3 = 0.f;
    for (; c + 4 * V <= dim; c += 4 * V) {          // four loads in flight, four independent accumulators
      const uint4 u0 = *reinterpret_cast<const uint4*>(kp + c), u1 = *reinterpret_cast<const uint4*>(kp + c + V),
                  u2 = *reinterpret_cast<const uint4*>(kp + c + 2 * V), u3 = *reinterpret_cast<const uint4*>(kp + c + 3 * V);
      float f0[V], f1[V], f2[V], f3[V];
      unpack<T>(u0, f0); unpack<T>(u1, f1); unpack<T>(u2, f2); unpack<T>(u3, f3);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        acc = fmaf(qs[c + i], f0[i], acc);
        a1 = fmaf(qs[c + V + i], f1[i], a1);
        a2 = fmaf(qs[c + 2 * V + i], f2[i], a2);
        a3 = fmaf(qs[c + 3 * V + i], f3[i], a3);
      }
    }
    for (; c < dim; c += V) {
      float f[V];
      unpack<T>(*reinterpret_cast<const uint4*>(kp + c), f);
#pragma unroll
      for (int i = 0; i < V; ++i) acc = fmaf(qs[c + i], f[i], acc);
    }
    acc += a1 + a2 + a3;
  } else {
    for (int c = 0; c < dim; ++c) acc = fmaf(qs[c], to_f<T>(kp[c]), acc);
  }
  return acc;
}

// DPL contiguous elements (4, 8 or 16 bytes, aligned: the caller checks the row width) as floats
template <typename T, int DPL>
__device__ __forceinline__ void load_cols(const T* __restrict__ src, float* f) {
  constexpr int BYTES = DPL * (int)sizeof(T);
  if constexpr (BYTES == 16) {
    const uint4 u = *reinterpret_cast<const uint4*>(src);
    if constexpr (sizeof(T) == 4) { f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y); f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w); }
    else unpack<T>(u, f);
  } else if constexpr (BYTES == 8) {
    const uint2 u = *reinterpret_cast<const uint2*>(src);
    if constexpr (sizeof(T) == 4) { f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y); }
    else { const T* t = reinterpret_cast<const T*>(&u); for (int i = 0; i < 4; ++i) f[i] = to_f<T>(t[i]); }
  } else if constexpr (BYTES == 4) {
    const uint32_t u = *reinterpret_cast<const uint32_t*>(src);
    if constexpr (sizeof(T) == 4) f[0] = __uint_as_float(u);
    else { const T* t = reinterpret_cast<const T*>(&u); f[0] = to_f<T>(t[0]); f[1] = to_f<T>(t[1]); }
  } else {
    for (int i = 0; i < DPL; ++i) f[i] = to_f<T>(src[i]);
  }
}

struct RagAttnParams {
  void* out; int ld_out;
  const void* q; int ld_q;
  const void* gate; int ld_gate;
  const void* k_pool; const void* v_pool;
  const int32_t* page_table; int pt_stride; int page_size;
  const int32_t* tok_slot; const int32_t* tok_pos;
  int n_tokens, H, G, dim, vdim;
  float scale; int window;
  const float* slopes;
  int keep_first;                // positions < keep_first stay visible behind the window
  int sigmoid_weights;           // 0: softmax over the visible keys; 1: weight = sigmoid(score + head_bias[h])
  const float* head_bias;        // per query head, added to the score (NULL: none)
  int gate_per_head;             // 0: gate[t][h * vdim + c]; 1: gate[t][h]
  float out_scale;
  int ld_k, ld_v;                // elements between the rows of the key / value pool (>= G * dim, G * vdim)
  const float* sink;             // per query head: exp(sink[h]) joins the softmax denominator (no key, no value)
  int chunk;                     // > 0: a key is visible only inside the query's block of `chunk` positions
  const float* out_rot;          // [vdim / 2]: the result is turned back by -position * out_rot[m] (rotated values)
  int out_rot_interleaved;       // pairs (2m, 2m + 1) instead of (m, m + vdim / 2)
};

// The visible keys of a token at position pos as one list: n_keep kept first positions, then [lo, pos].
struct KeyRange {
  int lo, n_keep, count;
  __device__ __forceinline__ KeyRange(int pos, int window, int keep_first, int chunk = 0) {
    lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (chunk > 0) lo = max(lo, pos / chunk * chunk);   // blocks are counted from position 0 of the sequence
    n_keep = min(max(keep_first, 0), lo);
    count = n_keep + pos - lo + 1;
  }
  __device__ __forceinline__ int key(int v) const { return v < n_keep ? v : lo + (v - n_keep); }
};

// Process keys [lo, hi] (inclusive) of one (token, head) for the calling warp; (m, l, acc) are the running state.
template <typename T, int DPL>
__device__ __forceinline__ void attend_range(const RagAttnParams& p, const float* qs, const int32_t* pt_row, int g,
                                             int pos, float slope, float bias, const KeyRange& kr, float& m, float& l,
                                             float* acc) {
  const int lo = 0, hi = kr.count - 1;              // virtual key indices
  const int lane = threadIdx.x & 31;
  const T* kpool = reinterpret_cast<const T*>(p.k_pool);
  const T* vpool = reinterpret_cast<const T*>(p.v_pool);
  const int kw = p.ld_k, vw = p.ld_v;
  for (int j0 = lo; j0 <= hi; j0 += 32) {
    const bool valid = j0 + lane <= hi;
    const int j = kr.key(j0 + lane);
    float s = -INFINITY;
    long long row = 0;
    if (valid) {
      row = (long long)pt_row[j / p.page_size] * p.page_size + j % p.page_size;
      s = dot_row<T>(qs, kpool + row * kw + g * p.dim, p.dim) * p.scale - slope * (float)(pos - j) + bias;
    }
    float m_new = m, pj;
    if (p.sigmoid_weights) {                       // unnormalised: no running maximum, m stays 0
      pj = valid ? 1.f / (1.f + expf(-s)) : 0.f;
      l += warp_sum(pj);
    } else {
      m_new = fmaxf(m, warp_max(s));
      const float corr = expf(m - m_new);          // m == -inf on the first block: exp(-inf) = 0
      pj = valid ? expf(s - m_new) : 0.f;
      l = l * corr + warp_sum(pj);
#pragma unroll
      for (int i = 0; i < DPL; ++i) acc[i] *= corr;
    }
    const int n = min(32, hi - j0 + 1);
    const bool vecv = p.vdim == 32 * DPL && DPL * sizeof(T) >= 4 && DPL * sizeof(T) <= 16 && vw % DPL == 0;   // lane = DPL contiguous columns
#pragma unroll 8
    for (int jj = 0; jj < n; ++jj) {
      const float w = __shfl_sync(0xffffffffu, pj, jj);
      const long long r = __shfl_sync(0xffffffffu, row, jj);
      const T* vp = vpool + r * vw + g * p.vdim + lane * DPL;
      if (vecv) {
        float f[DPL];
        load_cols<T, DPL>(vp, f);
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[i] = fmaf(w, f[i], acc[i]);
      } else {
#pragma unroll
        for (int i = 0; i < DPL; ++i)
          if (lane * DPL + i < p.vdim) acc[i] = fmaf(w, to_f<T>(vp[i]), acc[i]);
      }
    }
    m = m_new;
  }
}

// The pair partner of every column a lane owns, for turning the result back by the query's position: columns
// lane * DPL + i of the lanes of one warp.  Pairs that lie in one lane or at the same index of another lane take one
// shuffle at most; any other width walks the lane's DPL values.
template <int DPL>
__device__ __forceinline__ void rotate_back(const RagAttnParams& p, int t, float* val) {
  const int lane = threadIdx.x & 31, half = p.vdim >> 1;
  const float fpos = (float)p.tok_pos[t];
  float res[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int c = lane * DPL + i;
    const bool in = c < 2 * half;
    bool first;
    int pair, pc;
    if (p.out_rot_interleaved) { first = !(c & 1); pair = c >> 1; pc = c ^ 1; }
    else { first = c < half; pair = first ? c : c - half; pc = first ? c + half : c - half; }
    if (!in) pc = c;
    const int src_lane = pc / DPL, src_i = pc % DPL;
    float other = 0.f;
#pragma unroll
    for (int ii = 0; ii < DPL; ++ii) {
      const float s = __shfl_sync(0xffffffffu, val[ii], src_lane);
      if (ii == src_i) other = s;
    }
    float sn = 0.f, cs = 1.f;
    if (in) sincosf(-fpos * p.out_rot[pair], &sn, &cs);
    res[i] = in ? (first ? val[i] * cs - other * sn : val[i] * cs + other * sn) : val[i];
  }
#pragma unroll
  for (int i = 0; i < DPL; ++i) val[i] = res[i];
}

template <typename T, int DPL>
__device__ __forceinline__ void store_out(const RagAttnParams& p, int t, int h, float m, float l, const float* acc) {
  const int lane = threadIdx.x & 31;
  if (p.sink && !p.sigmoid_weights) l += expf(p.sink[h] - m);      // m: the maximum the sums are relative to
  T* o = reinterpret_cast<T*>(p.out) + (size_t)t * p.ld_out + h * p.vdim;
  const T* gt = (p.gate && !p.gate_per_head) ? reinterpret_cast<const T*>(p.gate) + (size_t)t * p.ld_gate + h * p.vdim : nullptr;
  float inv = (p.sigmoid_weights ? 1.f : 1.f / l) * p.out_scale;
  if (p.gate && p.gate_per_head)
    inv *= 1.f / (1.f + expf(-to_f<T>(reinterpret_cast<const T*>(p.gate)[(size_t)t * p.ld_gate + h])));
  float val[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) val[i] = acc[i] * inv;
  if (p.out_rot) rotate_back<DPL>(p, t, val);                      // before the gate: the gate is per column
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int c = lane * DPL + i;
    if (c < p.vdim) {
      float v = val[i];
      if (gt) v *= 1.f / (1.f + expf(-to_f<T>(gt[c])));
      o[c] = from_f<T>(v);
    }
  }
}

template <typename T, int DPL>
__global__ void __launch_bounds__(256) attention_ragged_kernel(RagAttnParams p) {
  extern __shared__ float smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const long long item = (long long)blockIdx.x * warps + warp;
  if (item >= (long long)p.n_tokens * p.H) return;
  const int t = (int)(item / p.H), h = (int)(item % p.H), g = h / (p.H / p.G);
  float* qs = smem + (size_t)warp * p.dim;
  const T* qr = reinterpret_cast<const T*>(p.q) + (size_t)t * p.ld_q + h * p.dim;
  for (int c = lane; c < p.dim; c += 32) qs[c] = to_f<T>(qr[c]);
  __syncwarp();
  const int pos = p.tok_pos[t];
  const int32_t* pt_row = p.page_table + (size_t)p.tok_slot[t] * p.pt_stride;
  const KeyRange kr(pos, p.window, p.keep_first, p.chunk);
  const float slope = p.slopes ? p.slopes[h] : 0.f, bias = p.head_bias ? p.head_bias[h] : 0.f;
  float m = p.sigmoid_weights ? 0.f : -INFINITY, l = 0.f, acc[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
  attend_range<T, DPL>(p, qs, pt_row, g, pos, slope, bias, kr, m, l, acc);
  store_out<T, DPL>(p, t, h, m, l, acc);
}

// R query rows against one key row: one pass over the key, R independent accumulators.
template <typename T, int R>
__device__ __forceinline__ void dot_rows(const float* __restrict__ qs, int dim, const T* __restrict__ kp, float* out) {
  constexpr int V = Vec<T>::N;
#pragma unroll
  for (int r = 0; r < R; ++r) out[r] = 0.f;
  if ((dim % V) == 0 && (reinterpret_cast<uintptr_t>(kp) & 15) == 0) {
#pragma unroll 2
    for (int c = 0; c < dim; c += V) {
      float f[V];
      unpack<T>(*reinterpret_cast<const uint4*>(kp + c), f);
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int i = 0; i < V; ++i) out[r] = fmaf(qs[r * dim + c + i], f[i], out[r]);
    }
  } else {
    for (int c = 0; c < dim; ++c) {
      const float kv = to_f<T>(kp[c]);
#pragma unroll
      for (int r = 0; r < R; ++r) out[r] = fmaf(qs[r * dim + c], kv, out[r]);
    }
  }
}

// One CTA per (token, key/value head, key slice): the R = H / G query heads that share the key/value head are
// handled together, so every key and value row is read once for all of them.  Warp w takes the key blocks w,
// w + warps, ... of its slice.  With one slice the CTA writes the output rows; with several it leaves (max, sum, acc)
// per query head in the workspace for the merge kernel.
template <typename T, int DPL, int R>
__global__ void __launch_bounds__(128) attention_ragged_split_kernel(RagAttnParams p, float* __restrict__ ws) {
  extern __shared__ float smem[];
  pdl_launch_dependents();
  pdl_wait();
  constexpr int PW = 2 + 32 * DPL;                     // floats of one partial
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  // R query heads per CTA: a key/value head's group of H / G query heads is cut into chunks of R (gv counts the chunks)
  const int chunks = p.H / (p.G * R), gv = blockIdx.x % (p.G * chunks);
  const int t = blockIdx.x / (p.G * chunks), g = gv / chunks, h0 = gv * R;
  float* qs = smem;                                    // [R][dim]
  float* part = smem + R * p.dim;                      // [warps][R][PW]
  const T* qr = reinterpret_cast<const T*>(p.q) + (size_t)t * p.ld_q + h0 * p.dim;
  for (int c = threadIdx.x; c < R * p.dim; c += blockDim.x) qs[c] = to_f<T>(qr[c]);
  __syncthreads();
  const int pos = p.tok_pos[t];
  const int32_t* pt_row = p.page_table + (size_t)p.tok_slot[t] * p.pt_stride;
  const KeyRange kr(pos, p.window, p.keep_first, p.chunk);
  float slope[R], bias[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    slope[r] = p.slopes ? p.slopes[h0 + r] : 0.f;
    bias[r] = p.head_bias ? p.head_bias[h0 + r] : 0.f;
  }
  const T* kpool = reinterpret_cast<const T*>(p.k_pool);
  const T* vpool = reinterpret_cast<const T*>(p.v_pool);
  const int kw = p.ld_k, vw = p.ld_v;
  const bool vecv = p.vdim == 32 * DPL && DPL * sizeof(T) >= 4 && DPL * sizeof(T) <= 16 && vw % DPL == 0;
  // this CTA's slice of the visible keys: whole 32-key blocks
  const int blocks = (kr.count + 31) / 32, per = (blocks + gridDim.y - 1) / gridDim.y;
  const int b_begin = blockIdx.y * per, b_end = min(blocks, b_begin + per);
  float m[R], l[R], acc[R][DPL];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    m[r] = p.sigmoid_weights ? 0.f : -INFINITY; l[r] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[r][i] = 0.f;
  }
  for (int b = b_begin + warp; b < b_end; b += warps) {
    const int j0 = 32 * b, hi = min(kr.count - 1, j0 + 31);
    const bool valid = j0 + lane <= hi;
    const int j = kr.key(j0 + lane);
    long long row = 0;
    float s[R], pj[R];
#pragma unroll
    for (int r = 0; r < R; ++r) s[r] = -INFINITY;
    if (valid) {
      row = (long long)pt_row[j / p.page_size] * p.page_size + j % p.page_size;
      dot_rows<T, R>(qs, p.dim, kpool + row * kw + g * p.dim, s);
#pragma unroll
      for (int r = 0; r < R; ++r) s[r] = s[r] * p.scale - slope[r] * (float)(pos - j) + bias[r];
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (p.sigmoid_weights) {
        pj[r] = valid ? 1.f / (1.f + expf(-s[r])) : 0.f;
        l[r] += warp_sum(pj[r]);
        continue;
      }
      const float m_new = fmaxf(m[r], warp_max(s[r]));
      const float corr = expf(m[r] - m_new);
      pj[r] = valid ? expf(s[r] - m_new) : 0.f;
      l[r] = l[r] * corr + warp_sum(pj[r]);
#pragma unroll
      for (int i = 0; i < DPL; ++i) acc[r][i] *= corr;
      m[r] = m_new;
    }
    const int n = hi - j0 + 1;
#pragma unroll 4
    for (int jj = 0; jj < n; ++jj) {
      const long long vr = __shfl_sync(0xffffffffu, row, jj);
      const T* vp = vpool + vr * vw + g * p.vdim + lane * DPL;
      float f[DPL];
      if (vecv) {
        load_cols<T, DPL>(vp, f);
      } else {
#pragma unroll
        for (int i = 0; i < DPL; ++i) f[i] = (lane * DPL + i < p.vdim) ? to_f<T>(vp[i]) : 0.f;
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float w = __shfl_sync(0xffffffffu, pj[r], jj);
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[r][i] = fmaf(w, f[i], acc[r][i]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float* mine = part + ((size_t)warp * R + r) * PW;
    if (lane == 0) { mine[0] = m[r]; mine[1] = l[r]; }
#pragma unroll
    for (int i = 0; i < DPL; ++i) mine[2 + lane * DPL + i] = acc[r][i];
  }
  __syncthreads();
  // warp r (and r + warps, ...) merges query head r over the warps, in warp order
  for (int r = warp; r < R; r += warps) {
    float M = -INFINITY;
    for (int w = 0; w < warps; ++w) M = fmaxf(M, part[((size_t)w * R + r) * PW]);
    float Lsum = 0.f, a[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) a[i] = 0.f;
    for (int w = 0; w < warps; ++w) {
      const float* pw = part + ((size_t)w * R + r) * PW;
      if (pw[1] == 0.f) continue;                       // this warp had no keys
      const float c = expf(pw[0] - M);
      Lsum += pw[1] * c;
#pragma unroll
      for (int i = 0; i < DPL; ++i) a[i] += pw[2 + lane * DPL + i] * c;
    }
    if (gridDim.y == 1) { store_out<T, DPL>(p, t, h0 + r, M, Lsum, a); continue; }
    float* o = ws + (((size_t)t * p.H + h0 + r) * gridDim.y + blockIdx.y) * PW;
    if (lane == 0) { o[0] = M; o[1] = Lsum; }
#pragma unroll
    for (int i = 0; i < DPL; ++i) o[2 + lane * DPL + i] = a[i];
  }
}

// One warp per (token, head): merges the key slices in slice order.
template <typename T, int DPL>
__global__ void attention_ragged_merge_kernel(RagAttnParams p, const float* __restrict__ ws, int slices) {
  pdl_launch_dependents();
  pdl_wait();
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= p.n_tokens * p.H) return;
  const float* base = ws + (size_t)item * slices * (2 + 32 * DPL);
  float M = -INFINITY;
  for (int s = 0; s < slices; ++s) M = fmaxf(M, base[(size_t)s * (2 + 32 * DPL)]);
  float Lsum = 0.f, acc[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
  for (int s = 0; s < slices; ++s) {
    const float* pw = base + (size_t)s * (2 + 32 * DPL);
    if (pw[1] == 0.f) continue;
    const float c = expf(pw[0] - M);
    Lsum += pw[1] * c;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] += pw[2 + lane * DPL + i] * c;
  }
  store_out<T, DPL>(p, item / p.H, item % p.H, M, Lsum, acc);
}

template <typename T, int DPL, int R>
static int launch_split(const RagAttnParams& p, float* ws, int slices, cudaStream_t st) {
  const int warps = 4;
  const size_t smem = sizeof(float) * ((size_t)R * p.dim + (size_t)warps * R * (2 + 32 * DPL));
  const long long items = (long long)p.n_tokens * p.H;
  int rc = launch_pdl("attention_ragged_split", attention_ragged_split_kernel<T, DPL, R>,
                      dim3((unsigned)(p.n_tokens * (p.H / R)), slices), dim3(warps * 32), smem, st, p, ws);
  if (rc != PG_OK || slices == 1) return rc;
  return launch_pdl("attention_ragged_merge", attention_ragged_merge_kernel<T, DPL>, dim3(cdiv(items, 4)), dim3(128), 0,
                    st, p, (const float*)ws, slices);
}

template <typename T, int DPL>
static int launch_ragged(const RagAttnParams& p, float* ws, long long ws_floats, cudaStream_t st) {
  const long long items = (long long)p.n_tokens * p.H;
  static const int split_max = env_int("PG_RAGGED_SPLIT_MAX_ITEMS", 592);   // below 4 (token, head) pairs per SM
  // query heads that one CTA serves from one read of the key / value rows: the largest of 8, 4, 2, 1 that divides the
  // group and keeps the accumulators (heads x value columns per lane) in registers
  const int group = p.H / p.G;
  int R = 1;
  for (int r = 8; r > 1; r >>= 1)
    if (group % r == 0 && r * DPL <= 64) { R = r; break; }
  if (items <= split_max && (p.window <= 0 || p.window > 64)) {
    // key slices until about two CTAs per SM are busy; a slice holds at least 128 keys (one block per warp)
    const long long ctas = (long long)p.n_tokens * (p.H / R);
    int span = p.window > 0 ? p.window : 1 << 20;
    if (p.chunk > 0) span = min(span, p.chunk);
    int slices = 1;
    while (slices < 32 && ctas * slices * 2 <= 296 && span / (slices * 2) >= 128 &&
           items * slices * 2 * (2 + 32 * DPL) <= ws_floats) slices *= 2;
    if (!ws) slices = 1;
    switch (R) {
      case 1: return launch_split<T, DPL, 1>(p, ws, slices, st);
      case 2: return launch_split<T, DPL, 2>(p, ws, slices, st);
      case 4: return launch_split<T, DPL, 4>(p, ws, slices, st);
      default: return launch_split<T, (DPL <= 8 ? DPL : 8), 8>(p, ws, slices, st);
    }
  }
  const int warps = 8;
  const size_t smem = sizeof(float) * (size_t)warps * p.dim;
  return launch_pdl("attention_ragged", attention_ragged_kernel<T, DPL>, dim3(cdiv(items, warps)), dim3(warps * 32), smem,
                    st, p);
}

}  // namespace pg

using namespace pg;

extern "C" int pg_attention_ragged_sink(void* out, int ld_out, const void* q, int ld_q, const void* gate, int ld_gate,
                                        int gate_per_head, const void* k_pool, int ld_k, const void* v_pool, int ld_v,
                                        const int32_t* page_table, int pt_stride, int page_size,
                                        const int32_t* tok_slot, const int32_t* tok_pos, int n_tokens, int n_heads,
                                        int n_kv_heads, int dim, int vdim, float scale, int window, int keep_first,
                                        const float* slopes, int sigmoid_weights, const float* head_bias,
                                        const float* sink, float out_scale, float* ws, long long ws_floats, int dtype,
                                        void* stream) {
  return pg_attention_ragged_masked(out, ld_out, q, ld_q, gate, ld_gate, gate_per_head, k_pool, ld_k, v_pool, ld_v, page_table,
                                    pt_stride, page_size, tok_slot, tok_pos, n_tokens, n_heads, n_kv_heads, dim, vdim, scale,
                                    window, keep_first, 0, slopes, sigmoid_weights, head_bias, sink, nullptr, 0, out_scale, ws,
                                    ws_floats, dtype, stream);
}

extern "C" int pg_attention_ragged_masked(void* out, int ld_out, const void* q, int ld_q, const void* gate, int ld_gate,
                                          int gate_per_head, const void* k_pool, int ld_k, const void* v_pool, int ld_v,
                                          const int32_t* page_table, int pt_stride, int page_size,
                                          const int32_t* tok_slot, const int32_t* tok_pos, int n_tokens, int n_heads,
                                          int n_kv_heads, int dim, int vdim, float scale, int window, int keep_first,
                                          int chunk, const float* slopes, int sigmoid_weights, const float* head_bias,
                                          const float* sink, const float* out_rot, int out_rot_interleaved,
                                          float out_scale, float* ws, long long ws_floats, int dtype, void* stream) {
  if (n_tokens <= 0) return PG_OK;
  PG_REQUIRE(chunk >= 0 && (chunk == 0 || keep_first == 0), "attention_ragged: blocks of %d positions with %d kept first ones",
             chunk, keep_first);
  if (ld_k <= 0) ld_k = n_kv_heads * dim;
  if (ld_v <= 0) ld_v = n_kv_heads * vdim;
  PG_REQUIRE(ld_k >= n_kv_heads * dim && ld_v >= n_kv_heads * vdim, "attention_ragged: pool rows of %d / %d elements", ld_k, ld_v);
  PG_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "attention_ragged: heads %d / kv heads %d",
             n_heads, n_kv_heads);
  PG_REQUIRE(dim > 0 && dim <= 1024 && vdim > 0 && vdim <= 512, "attention_ragged: dim %d (<= 1024), vdim %d (<= 512)", dim, vdim);
  RagAttnParams p = {out, ld_out, q, ld_q, gate, ld_gate, k_pool, v_pool, page_table, pt_stride, page_size, tok_slot,
                     tok_pos, n_tokens, n_heads, n_kv_heads, dim, vdim, scale, window, slopes, keep_first,
                     sigmoid_weights ? 1 : 0, head_bias, gate_per_head ? 1 : 0, out_scale, ld_k, ld_v, sink, chunk, out_rot,
                     out_rot_interleaved ? 1 : 0};
  cudaStream_t st = (cudaStream_t)stream;
  const int dpl = (vdim + 31) / 32;
  PG_DISPATCH_DTYPE(dtype, T, {
    if (dpl <= 1) return launch_ragged<T, 1>(p, ws, ws_floats, st);
    if (dpl <= 2) return launch_ragged<T, 2>(p, ws, ws_floats, st);
    if (dpl <= 4) return launch_ragged<T, 4>(p, ws, ws_floats, st);
    if (dpl <= 8) return launch_ragged<T, 8>(p, ws, ws_floats, st);
    return launch_ragged<T, 16>(p, ws, ws_floats, st);
  });
  return PG_OK;
}

extern "C" int pg_attention_ragged_ex(void* out, int ld_out, const void* q, int ld_q, const void* gate, int ld_gate,
                                      int gate_per_head, const void* k_pool, const void* v_pool,
                                      const int32_t* page_table, int pt_stride, int page_size, const int32_t* tok_slot,
                                      const int32_t* tok_pos, int n_tokens, int n_heads, int n_kv_heads, int dim,
                                      int vdim, float scale, int window, int keep_first, const float* slopes,
                                      int sigmoid_weights, const float* head_bias, float out_scale, float* ws,
                                      long long ws_floats, int dtype, void* stream) {
  return pg_attention_ragged_sink(out, ld_out, q, ld_q, gate, ld_gate, gate_per_head, k_pool, 0, v_pool, 0, page_table,
                                  pt_stride, page_size, tok_slot, tok_pos, n_tokens, n_heads, n_kv_heads, dim, vdim, scale,
                                  window, keep_first, slopes, sigmoid_weights, head_bias, nullptr, out_scale, ws, ws_floats,
                                  dtype, stream);
}

extern "C" int pg_attention_ragged(void* out, int ld_out, const void* q, int ld_q, const void* gate, int ld_gate,
                                   const void* k_pool, const void* v_pool, const int32_t* page_table, int pt_stride,
                                   int page_size, const int32_t* tok_slot, const int32_t* tok_pos, int n_tokens,
                                   int n_heads, int n_kv_heads, int dim, int vdim, float scale, int window,
                                   const float* slopes, float* ws, long long ws_floats, int dtype, void* stream) {
  return pg_attention_ragged_ex(out, ld_out, q, ld_q, gate, ld_gate, 0, k_pool, v_pool, page_table, pt_stride, page_size,
                                tok_slot, tok_pos, n_tokens, n_heads, n_kv_heads, dim, vdim, scale, window, 0, slopes, 0,
                                nullptr, 1.f, ws, ws_floats, dtype, stream);
}
