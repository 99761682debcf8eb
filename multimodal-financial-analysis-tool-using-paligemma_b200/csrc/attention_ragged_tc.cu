// Windowed causal attention with distance bias for ragged token batches on the tcgen05 tensor cores (prompt portions).
//
// The step's tokens are cut on the host into query tiles: up to 128 consecutive tokens of ONE sequence at consecutive
// positions (tile = {first token row, rows, page-table row, first position}).  One CTA = one (tile, head).  The keys a
// tile can see are the positions [max(0, pos0 - window + 1), pos0 + rows - 1] of its sequence, walked page by page
// (key tile = page = 64 keys, fetched by TMA from the paged pools; the append kernel has written the step's own keys
// before this launch).  Two passes over the key tiles, both on the tensor cores, as in attention_tc.cu:
//   pass 0: S = Q K^T (tcgen05.mma, fp32 in TMEM) -> thread r owns query row r: s = S * scale - slope_h * (i - j),
//           masked outside 0 <= i - j < window, running row maximum (no shuffles);
//   pass 1: S again (K double-buffered, V in one buffer), p = exp(s - max) in fp32, row sum from the fp32 values, P rounded to the model dtype into a
//           K-major SWIZZLE_128B tile, O += P V with V as an MN-major operand straight from its [key, vdim] page.
// Epilogue: O / sum, times sigmoid(gate), rounded once.  Key width and value width are independent multiples of 64.
// Extensions (pg_attention_ragged_tc_ex): keep_first > 0 keeps the first keep_first positions visible behind the
// window: the key tiles are then the pages that hold them (as far as they lie before the window's first page)
// followed by the window's pages.  sigmoid_weights: ONE pass, p = sigmoid(s + head_bias[h]), no maximum, no sum.  The
// gate may be one value per (token, head); the result is multiplied by out_scale before it is rounded.
// Every mbarrier wait is bounded: a wait that gives up sets the error flag, the roles leave their loops, the CTA lets
// its copies land, frees its TMEM and returns.
#include <cmath>

#include "tc_common.cuh"

namespace pg {
namespace tc {

constexpr int WQ = 128;   // query rows per CTA == TMEM lanes
constexpr int WK = 64;    // keys per tile == page size

__device__ __forceinline__ uint64_t umma_desc_mn_w(uint32_t smem_addr, uint32_t lbo_bytes) {
  // MN-major, SWIZZLE_128B: 64 contiguous MN elements (128 B) per K row, 8-row groups 1024 B apart (SBO),
  // next 64-element MN block lbo_bytes away (LBO)
  return (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) | (64ull << 32) |
         (1ull << 46) | (2ull << 61);
}

constexpr uint32_t W_WAIT_LIMIT = 1u << 22;
__device__ __forceinline__ bool wait_lim(uint32_t bar, uint32_t parity, volatile int* fail) {
  for (uint32_t it = 0; it < W_WAIT_LIMIT; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 255u && *fail) return false;
  }
  *fail = 1;
  return false;
}

struct WinParams {
  void* out; int ld_out;
  const void* gate; int ld_gate;
  const int32_t* tiles;          // [n_tiles][4] = {token row0, rows, page-table row, position of row0}
  const int32_t* page_table; int pt_stride;
  int H, kv_group, dim, vdim;
  float scale; int window;
  const float* slopes;
  int* err_flag;
  int keep_first, sigmoid_weights;
  const float* head_bias;
  int gate_per_head;
  float out_scale;
  const float* sink;             // per query head: exp(sink[h]) joins the softmax denominator (NULL: none)
  int chunk;                     // > 0: a key is visible only inside the query's block of `chunk` positions
  const float* out_rot;          // [vdim / 2]: the result is turned back by -position * out_rot[m] (rotated values)
  int out_rot_interleaved;       // pairs (2m, 2m + 1) instead of (m, m + vdim / 2)
};

template <typename T>
__global__ void __launch_bounds__(256, 1)
attention_window_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                           const __grid_constant__ CUtensorMap map_v, WinParams p) {
  constexpr int FMT = std::is_same<T, bf16>::value ? 1 : 0;
  const int KB = p.dim / 64, VB = p.vdim / 64;
  const int Q_BYTES = WQ * p.dim * 2, K_BYTES = WK * p.dim * 2, V_BYTES = WK * p.vdim * 2, P_BYTES = WQ * WK * 2;
  const int S_COL = 0, O_COL = WK;
  const int tmem_cols = (WK + p.vdim <= 256) ? 256 : 512;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // K tiles are double-buffered (tile it+1 is requested as soon as S(it) has been issued); V has ONE buffer, requested
  // when the previous P V has finished and hidden behind S and the softmax of its own tile: 99 KB at 128-wide heads,
  // so that two CTAs share an SM and overlap each other's load -> MMA -> softmax -> MMA chains
  const uint32_t s_q = base, s_k0 = s_q + Q_BYTES, s_vb = s_k0 + 2 * K_BYTES, s_p = s_vb + V_BYTES;
  auto s_k = [&](int bf) { return s_k0 + bf * K_BYTES; };
  const uint32_t bars = s_p + P_BYTES;
  const uint32_t bar_q = bars, bar_kv0 = bars + 8, bar_s = bars + 16, bar_sfree = bars + 24, bar_p = bars + 32,
                 bar_o = bars + 40, bar_kv1 = bars + 48, bar_v = bars + 56, tmem_slot = bars + 64;
  auto bar_kv = [&](int bf) { return bf ? bar_kv1 : bar_kv0; };
  uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));
  uint8_t* p_ptr = smem_raw + (s_p - smem_u32(smem_raw));
  __shared__ int s_fail;
  volatile int* fail = &s_fail;
  if (threadIdx.x == 0) s_fail = 0;

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, kvh = h / p.kv_group;

  if (warp == 1 && lane == 0) {
    mbar_init(bar_q, 1); mbar_init(bar_kv0, 1); mbar_init(bar_kv1, 1); mbar_init(bar_s, 1); mbar_init(bar_sfree, 128);
    mbar_init(bar_p, 128); mbar_init(bar_o, 1); mbar_init(bar_v, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  pdl_wait();  // q, the pools, the tile list and the page table come from the preceding kernels / copies
  const int32_t* tile = p.tiles + 4 * (size_t)blockIdx.x;
  const int row0 = tile[0], rows = tile[1], slot = tile[2], pos0 = tile[3];
  const int hi = pos0 + rows - 1;                                        // last key position any row can see
  int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;               // first one
  if (p.chunk > 0) lo = max(lo, pos0 / p.chunk * p.chunk);               // the block of the tile's first row
  const int t_lo = lo / WK;
  // pages of the kept first positions that lie before the window's first page, then the window's pages
  const int n_keep = (p.keep_first > 0 && p.window > 0) ? min((p.keep_first + WK - 1) / WK, t_lo) : 0;
  const int n_tiles = n_keep + hi / WK - t_lo + 1;
  auto page_of = [&](int t) { return t < n_keep ? t : t_lo + (t - n_keep); };   // key tile -> page of the sequence
  const int32_t* pt_row = p.page_table + (size_t)slot * p.pt_stride;
  const bool sig = p.sigmoid_weights != 0;

  if (warp == 0 && lane == 0) {
    // ===================== TMA + MMA issuer (one thread) =====================
    const uint32_t idesc_s = umma_idesc(FMT, WQ, WK);
    const uint32_t idesc_o = umma_idesc(FMT, WQ, p.vdim) | (1u << 16);  // B (= V) is MN-major
    mbar_expect_tx(bar_q, Q_BYTES);
    for (int kb = 0; kb < KB; ++kb)
      tma_load_2d(s_q + kb * (WQ * 128), &map_q, bar_q, h * p.dim + kb * 64, row0);
    const int total = sig ? n_tiles : 2 * n_tiles;
    auto request = [&](int i) {   // K of flat step i into K buffer i & 1
      const int t = page_of(i >= n_tiles ? i - n_tiles : i), bf = i & 1;
      const int row = pt_row[t] * WK;
      mbar_expect_tx(bar_kv(bf), K_BYTES);
      for (int kb = 0; kb < KB; ++kb)
        tma_load_2d(s_k(bf) + kb * (WK * 128), &map_k, bar_kv(bf), kvh * p.dim + kb * 64, row);
    };
    auto request_v = [&](int t) {   // V of key tile t (pass 1) into the V buffer
      const int row = pt_row[page_of(t)] * WK;
      mbar_expect_tx(bar_v, V_BYTES);
      for (int vb = 0; vb < VB; ++vb)
        tma_load_2d(s_vb + vb * (WK * 128), &map_v, bar_v, kvh * p.vdim + vb * 64, row);
    };
    request(0);
    if (!wait_lim(bar_q, 0, fail)) goto issuer_done;
    for (int it = 0; it < total; ++it) {
      const int pass = (sig || it >= n_tiles) ? 1 : 0, t = it >= n_tiles ? it - n_tiles : it, bf = it & 1;
      if (it > 0 && !wait_lim(bar_sfree, (it - 1) & 1, fail)) goto issuer_done;          // S of the previous tile was read
      if (pass == 1 && t > 0 && !wait_lim(bar_o, (t - 1) & 1, fail)) goto issuer_done;   // previous PV done with V and P
      if (pass == 1) request_v(t);                                 // lands behind S(it) and the softmax of this tile
      if (!wait_lim(bar_kv(bf), (it >> 1) & 1, fail)) goto issuer_done;
      tc_fence_after();
      for (int ks = 0; ks < p.dim / 16; ++ks) {                    // S = Q K^T
        const uint32_t off_q = (ks / 4) * (WQ * 128) + (ks % 4) * 32, off_k = (ks / 4) * (WK * 128) + (ks % 4) * 32;
        umma(tmem_base + S_COL, umma_desc(s_q + off_q), umma_desc(s_k(bf) + off_k), idesc_s, ks > 0 ? 1u : 0u);
      }
      umma_commit(bar_s);
      if (it + 1 < total) request(it + 1);                         // the other K buffer is free (bar_sfree above)
      if (pass == 1) {
        if (!wait_lim(bar_p, t & 1, fail)) goto issuer_done;       // P tile is in shared memory
        if (!wait_lim(bar_v, t & 1, fail)) goto issuer_done;       // and so is V
        tc_fence_after();
        for (int ks = 0; ks < WK / 16; ++ks) {                     // O += P V
          umma(tmem_base + O_COL, umma_desc(s_p + ks * 32), umma_desc_mn_w(s_vb + ks * 2048, WK * 128), idesc_o,
               (t > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(bar_o);
      }
    }
  issuer_done:;
  } else if (warp >= 4) {
    // ===================== softmax + epilogue: thread <-> query row =====================
    const int qw = warp & 3, r = qw * 32 + lane;
    const uint32_t t_row = tmem_base + ((uint32_t)(qw * 32) << 16);
    const int i = pos0 + r;                                        // this row's position
    const float slope = p.slopes ? p.slopes[h] : 0.f, hbias = p.head_bias ? p.head_bias[h] : 0.f;
    const int blk0 = p.chunk > 0 ? i / p.chunk * p.chunk : 0;      // first position of this row's block
    float m = -INFINITY, l = 0.f;
    int it = 0;
    bool ok = true;
    for (int pass = sig ? 1 : 0; pass < 2 && ok; ++pass) {
      for (int t = 0; t < n_tiles; ++t, ++it) {
        if (!wait_lim(bar_s, it & 1, fail)) { ok = false; break; }
        tc_fence_after();
        if (pass == 1 && t > 0 && !wait_lim(bar_o, (t - 1) & 1, fail)) { ok = false; break; }   // P buffer is free again
        const int j0 = page_of(t) * WK;
#pragma unroll 1
        for (int c = 0; c < WK / 32; ++c) {
          float s[32];
          tmem_ld32(t_row + S_COL + c * 32, s);
          tmem_ld_wait();
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) {
            const int j = j0 + c * 32 + jj, back = i - j;
            const bool vis = back >= 0 && j >= blk0 && (p.window <= 0 || back < p.window || j < p.keep_first);
            s[jj] = vis ? s[jj] * p.scale - slope * (float)back + hbias : -INFINITY;
          }
          if (pass == 0) {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) m = fmaxf(m, s[jj]);
          } else {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) {
              s[jj] = sig ? 1.f / (1.f + __expf(-s[jj])) : __expf(s[jj] - m);   // exp(+inf) -> weight 0 when masked
              l += s[jj];
            }
            // P[r][c*32 .. +31] into the K-major SWIZZLE_128B tile (128 rows x 128 B)
            uint8_t* blk = p_ptr + r * 128;
#pragma unroll
            for (int q0 = 0; q0 < 32; q0 += 8) {
              const int chunk = (c * 4 + q0 / 8) ^ (r & 7);
              *reinterpret_cast<uint4*>(blk + chunk * 16) = pack<T>(s + q0);
            }
          }
        }
        tc_fence_before();
        if (pass == 1) {
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy smem writes -> UMMA
          mbar_arrive(bar_p);
        }
        mbar_arrive(bar_sfree);
      }
    }
    if (ok && wait_lim(bar_o, (n_tiles - 1) & 1, fail)) {
      tc_fence_after();
      if (p.sink && !sig) l += __expf(p.sink[h] - m);              // a logit without key or value, counted once
      float inv = (sig ? 1.f : 1.f / l) * p.out_scale;
      const size_t trow = (size_t)row0 + r;
      T* orow = reinterpret_cast<T*>(p.out) + trow * p.ld_out + (size_t)h * p.vdim;
      const T* grow = (p.gate && !p.gate_per_head) ? reinterpret_cast<const T*>(p.gate) + trow * p.ld_gate + (size_t)h * p.vdim : nullptr;
      if (p.gate && p.gate_per_head && r < rows)
        inv *= 1.f / (1.f + __expf(-to_f<T>(reinterpret_cast<const T*>(p.gate)[trow * p.ld_gate + h])));
      auto store32 = [&](int c, const float* o) {                  // 32 finished columns of this row: gate, round, store
        if (r >= rows) return;
#pragma unroll
        for (int q0 = 0; q0 < 32; q0 += 8) {
          float w[8], gt[8];
          if (grow) unpack<T>(*reinterpret_cast<const uint4*>(grow + c * 32 + q0), gt);
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) {
            float v = o[q0 + jj];
            if (grow) v *= 1.f / (1.f + __expf(-gt[jj]));
            w[jj] = v;
          }
          *reinterpret_cast<uint4*>(orow + c * 32 + q0) = pack<T>(w);
        }
      };
      const float fpos = (float)i;
      if (!p.out_rot) {
#pragma unroll 1
        for (int c = 0; c * 32 < p.vdim; ++c) {
          float o[32];
          tmem_ld32(t_row + O_COL + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) o[jj] *= inv;
          store32(c, o);
        }
      } else if (p.out_rot_interleaved) {                          // pairs of neighbours: both halves in one load
#pragma unroll 1
        for (int c = 0; c * 32 < p.vdim; ++c) {
          float o[32];
          tmem_ld32(t_row + O_COL + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            float sn, cs;
            sincosf(-fpos * p.out_rot[c * 16 + k], &sn, &cs);
            const float u = o[2 * k] * inv, v = o[2 * k + 1] * inv;
            o[2 * k] = u * cs - v * sn;
            o[2 * k + 1] = v * cs + u * sn;
          }
          store32(c, o);
        }
      } else {                                                     // column m with m + vdim / 2 (vdim is a multiple of 64)
        const int hc = p.vdim / 64;
#pragma unroll 1
        for (int c = 0; c < hc; ++c) {
          float a[32], b[32];
          tmem_ld32(t_row + O_COL + c * 32, a);
          tmem_ld32(t_row + O_COL + (hc + c) * 32, b);
          tmem_ld_wait();
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) {
            float sn, cs;
            sincosf(-fpos * p.out_rot[c * 32 + jj], &sn, &cs);
            const float u = a[jj] * inv, v = b[jj] * inv;
            a[jj] = u * cs - v * sn;
            b[jj] = v * cs + u * sn;
          }
          store32(c, a);
          store32(hc + c, b);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (s_fail) {  // let copies and MMAs that are still in flight finish before the shared memory and TMEM go away
    for (int k = 0; k < 2000; ++k) __nanosleep(1000);
    if (threadIdx.x == 0 && p.err_flag) *p.err_flag = 2;
    __syncthreads();
  }
  if (warp == 2) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

}  // namespace tc
}  // namespace pg

using namespace pg;

extern "C" int pg_attention_ragged_tc_ok(int dim, int vdim, int page_size, int ld_q, int ld_out, int ld_gate, int dtype) {
  static const int enabled = env_int("PG_RAGGED_ATTN_TC", 1);
  if (!enabled || (dtype != PG_BF16 && dtype != PG_F16) || page_size != tc::WK) return 0;
  if (dim % 64 || vdim % 64 || dim > 256 || vdim > 256 || ld_q % 8 || ld_out % 8 || ld_gate % 8) return 0;
  return tc::encode_fn() != nullptr ? 1 : 0;
}

extern "C" int pg_attention_ragged_tc_sink(void* out, int ld_out, const void* q, int ld_q, const void* gate, int ld_gate,
                                           int gate_per_head, const void* k_pool, int ld_k, const void* v_pool, int ld_v,
                                           long long pool_rows, const int32_t* page_table, int pt_stride, int page_size,
                                           const int32_t* tiles, int n_tiles, int n_tokens, int n_heads, int n_kv_heads,
                                           int dim, int vdim, float scale, int window, int keep_first,
                                           const float* slopes, int sigmoid_weights, const float* head_bias,
                                           const float* sink, float out_scale, int* err_flag, int dtype, void* stream) {
  return pg_attention_ragged_tc_masked(out, ld_out, q, ld_q, gate, ld_gate, gate_per_head, k_pool, ld_k, v_pool, ld_v, pool_rows,
                                       page_table, pt_stride, page_size, tiles, n_tiles, n_tokens, n_heads, n_kv_heads, dim,
                                       vdim, scale, window, keep_first, 0, slopes, sigmoid_weights, head_bias, sink, nullptr, 0,
                                       out_scale, err_flag, dtype, stream);
}

extern "C" int pg_attention_ragged_tc_masked(void* out, int ld_out, const void* q, int ld_q, const void* gate, int ld_gate,
                                             int gate_per_head, const void* k_pool, int ld_k, const void* v_pool, int ld_v,
                                             long long pool_rows, const int32_t* page_table, int pt_stride, int page_size,
                                             const int32_t* tiles, int n_tiles, int n_tokens, int n_heads, int n_kv_heads,
                                             int dim, int vdim, float scale, int window, int keep_first, int chunk,
                                             const float* slopes, int sigmoid_weights, const float* head_bias,
                                             const float* sink, const float* out_rot, int out_rot_interleaved,
                                             float out_scale, int* err_flag, int dtype, void* stream) {
  if (n_tiles <= 0) return PG_OK;
  PG_REQUIRE(chunk >= 0 && (chunk == 0 || keep_first == 0), "attention_ragged_tc: blocks of %d positions with %d kept first ones",
             chunk, keep_first);
  if (ld_k <= 0) ld_k = n_kv_heads * dim;
  if (ld_v <= 0) ld_v = n_kv_heads * vdim;
  PG_REQUIRE(ld_k >= n_kv_heads * dim && ld_v >= n_kv_heads * vdim && ld_k % 8 == 0 && ld_v % 8 == 0,
             "attention_ragged_tc: pool rows of %d / %d elements", ld_k, ld_v);
  PG_REQUIRE(pg_attention_ragged_tc_ok(dim, vdim, page_size, ld_q, ld_out, (gate && !gate_per_head) ? ld_gate : 8, dtype),
             "attention_ragged_tc: unsupported problem (dim %d vdim %d page %d dtype %d)", dim, vdim, page_size, dtype);
  PG_REQUIRE(n_heads % n_kv_heads == 0, "attention_ragged_tc: heads %d / kv heads %d", n_heads, n_kv_heads);
  PG_REQUIRE(((uintptr_t)q % 16) == 0 && ((uintptr_t)out % 16) == 0 && (gate_per_head || ((uintptr_t)gate % 16) == 0) &&
                 ((uintptr_t)k_pool % 16) == 0 && ((uintptr_t)v_pool % 16) == 0,
             "attention_ragged_tc: operands must be 16-byte aligned");
  const bool bf = dtype == PG_BF16;
  CUtensorMap mq, mk, mv;
  PG_REQUIRE(tc::make_map_2d(&mq, q, n_tokens, (long long)n_heads * dim, ld_q, tc::WQ, bf) &&
                 tc::make_map_2d(&mk, k_pool, pool_rows, (long long)n_kv_heads * dim, (long long)ld_k, tc::WK, bf) &&
                 tc::make_map_2d(&mv, v_pool, pool_rows, (long long)n_kv_heads * vdim, (long long)ld_v, tc::WK, bf),
             "attention_ragged_tc: cuTensorMapEncodeTiled failed");
  tc::WinParams p = {out, ld_out, gate, ld_gate, tiles, page_table, pt_stride, n_heads, n_heads / n_kv_heads, dim, vdim,
                     scale, window, slopes, err_flag, keep_first, sigmoid_weights ? 1 : 0, head_bias,
                     gate_per_head ? 1 : 0, out_scale, sink, chunk, out_rot, out_rot_interleaved ? 1 : 0};
  const size_t smem = 1024 + (size_t)tc::WQ * dim * 2 + 2 * (size_t)tc::WK * dim * 2 + (size_t)tc::WK * vdim * 2 +
                      (size_t)tc::WQ * tc::WK * 2 + 72 + 16;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(n_tiles, n_heads);
  if (bf) {
    auto kern = tc::attention_window_tc_kernel<bf16>;
    PG_REQUIRE(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess,
               "attention_ragged_tc: cannot reserve %zu B of shared memory", smem);
    return launch_tc("attention_ragged_tc", kern, grid, dim3(256), smem, 1, false, st, mq, mk, mv, p);
  }
  auto kern = tc::attention_window_tc_kernel<f16>;
  PG_REQUIRE(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess,
             "attention_ragged_tc: cannot reserve %zu B of shared memory", smem);
  return launch_tc("attention_ragged_tc", kern, grid, dim3(256), smem, 1, false, st, mq, mk, mv, p);
}

extern "C" int pg_attention_ragged_tc_ex(void* out, int ld_out, const void* q, int ld_q, const void* gate, int ld_gate,
                                         int gate_per_head, const void* k_pool, const void* v_pool, long long pool_rows,
                                         const int32_t* page_table, int pt_stride, int page_size, const int32_t* tiles,
                                         int n_tiles, int n_tokens, int n_heads, int n_kv_heads, int dim, int vdim,
                                         float scale, int window, int keep_first, const float* slopes,
                                         int sigmoid_weights, const float* head_bias, float out_scale, int* err_flag,
                                         int dtype, void* stream) {
  return pg_attention_ragged_tc_sink(out, ld_out, q, ld_q, gate, ld_gate, gate_per_head, k_pool, 0, v_pool, 0, pool_rows,
                                     page_table, pt_stride, page_size, tiles, n_tiles, n_tokens, n_heads, n_kv_heads, dim,
                                     vdim, scale, window, keep_first, slopes, sigmoid_weights, head_bias, nullptr, out_scale,
                                     err_flag, dtype, stream);
}

extern "C" int pg_attention_ragged_tc(void* out, int ld_out, const void* q, int ld_q, const void* gate, int ld_gate,
                                      const void* k_pool, const void* v_pool, long long pool_rows,
                                      const int32_t* page_table, int pt_stride, int page_size, const int32_t* tiles,
                                      int n_tiles, int n_tokens, int n_heads, int n_kv_heads, int dim, int vdim,
                                      float scale, int window, const float* slopes, int* err_flag, int dtype,
                                      void* stream) {
  return pg_attention_ragged_tc_ex(out, ld_out, q, ld_q, gate, ld_gate, 0, k_pool, v_pool, pool_rows, page_table, pt_stride,
                                   page_size, tiles, n_tiles, n_tokens, n_heads, n_kv_heads, dim, vdim, scale, window, 0,
                                   slopes, 0, nullptr, 1.f, err_flag, dtype, stream);
}
