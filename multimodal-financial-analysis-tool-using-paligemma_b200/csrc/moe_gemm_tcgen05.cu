// Grouped expert GEMM on the 5th-generation tensor cores: out[pos] = A[pos] W_e^T for the rows of every expert e
// (offsets[e] <= pos < offsets[e+1], rows already grouped by expert), optionally with the SwiGLU pairing of
// stacked [Wg; Wu] weights.  Same machinery as gemm_tcgen05.cu -- persistent, warp-specialised, one CTA per SM:
//   warp 0  TMA producer      ring of NSTAGES x {A 128x64, W BNx64 [, W_up BNx64]} (SWIZZLE_128B)
//   warp 1  MMA issuer        tcgen05.mma cta_group::1 kind::f16, M=128 x N=BN x K=16, fp32 accumulators in TMEM
//   warp 2  TMEM allocator    2 accumulator stages
//   warps 4-7 epilogue        tcgen05.ld -> (silu(g) * u) -> rounded rows to global
// What differs is the tile scheduler: the number of rows per expert is only known on the device, so every role walks
// the same tile sequence from the offsets array: expert e owns ceil(rows_e / 128) x ceil(N / BN) tiles, numbered
// expert by expert, n-block major inside an expert (neighbouring CTAs share the weight tile through L2).  A tile's
// A rows are one TMA box at row offsets[e] + 128 * m_blk of the grouped activations; rows past the expert's end
// belong to the next expert (or are zero fill) and are masked in the epilogue.  The weights of all experts are ONE
// 2-D tensor map over [n_experts * rows_per_expert, K].
#include "tc_common.cuh"

namespace pg {
namespace tc {

constexpr int MG_BM = 128, MG_BK = 64, MG_UMMA_K = 16, MG_THREADS = 256, MG_TMEM_COLS = 512;
constexpr int MG_A_BYTES = MG_BM * MG_BK * 2;

struct MoeParams {
  void* out;
  const int32_t* offsets;
  int n_experts, N, K, ldo;
  int* err_flag;   // device-visible int, set to 2 when a pipeline wait gave up (may be NULL)
  int act;         // pairing of the two products of a stacked [Wg; Wu] tile: PG_GLU_SILU or PG_GLU_CLAMPED
  float limit;     // PG_GLU_CLAMPED: g' = min(g, limit), u' = clamp(u, -limit, limit), g' sigmoid(1.702 g') (u' + 1)
  // Per-head mode (group_rows > 0; offsets unused): every group is one head of the SAME group_rows token rows.  Group e
  // reads its operand at columns e * a_gs of the token rows (the A map covers the token-major matrix) and writes
  // columns e * o_gs of them.
  int group_rows, a_gs, o_gs;
};

// Every wait of this kernel is bounded: if the roles ever disagreed about the tile sequence (the offsets are data),
// a barrier would never complete.  The first wait that runs out sets the CTA's flag; every later wait returns at
// once, the roles leave their loops, the CTA lets its copies in flight land, frees its TMEM and returns, and the
// host finds the error flag.
constexpr uint32_t MG_WAIT_LIMIT = 1u << 22;
__device__ __forceinline__ bool mbar_wait_lim(uint32_t bar, uint32_t parity, volatile int* fail) {
  for (uint32_t it = 0; it < MG_WAIT_LIMIT; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 255u && *fail) return false;
  }
  *fail = 1;
  return false;
}

// Walks the tile sequence; every role owns one cursor and asks for increasing tile numbers.
struct TileCursor {
  const int32_t* off;
  int n_experts, n_tiles_n, e, first;   // first = number of the first tile of expert e
  int fixed;                            // > 0: every group has this many rows (off is not read)
  __device__ __forceinline__ TileCursor(const int32_t* o, int ne, int ntn, int fx = 0)
      : off(o), n_experts(ne), n_tiles_n(ntn), e(0), first(0), fixed(fx) {}
  __device__ __forceinline__ int at(int i) const { return fixed > 0 ? i * fixed : off[i]; }
  // -> false when the sequence is exhausted
  __device__ __forceinline__ bool seek(int tile, int& expert, int& m0, int& m_end, int& n_blk) {
    while (e < n_experts) {
      const int rows = at(e + 1) - at(e);
      const int mt = (rows + MG_BM - 1) / MG_BM;
      const int cnt = mt * n_tiles_n;
      if (tile < first + cnt) {
        const int i = tile - first;
        expert = e;
        n_blk = i / mt;
        m0 = at(e) + (i % mt) * MG_BM;
        m_end = at(e + 1);
        return true;
      }
      first += cnt;
      ++e;
    }
    return false;
  }
};

template <typename T, bool DUAL, int BN>
__global__ void __launch_bounds__(MG_THREADS, 1)
moe_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, MoeParams p) {
  constexpr int NB_TILES = DUAL ? 2 : 1;
  constexpr int NSTAGES = (DUAL && BN > 64) ? 4 : 6;
  constexpr int W_BYTES = BN * MG_BK * 2;
  constexpr int STAGE_BYTES = MG_A_BYTES + NB_TILES * W_BYTES;
  constexpr int ACC_COLS = NB_TILES * BN;
  constexpr uint32_t IDESC = umma_idesc(std::is_same<T, bf16>::value ? 1 : 0, MG_BM, BN);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = smem_base + NSTAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (NSTAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * NSTAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * NSTAGES + 2 + a); };
  const uint32_t tmem_slot = bars + 8u * (2 * NSTAGES + 4);
  uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  __shared__ int s_fail;
  volatile int* fail = &s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles_n = (p.N + BN - 1) / BN;
  const int k_blocks = (p.K + MG_BK - 1) / MG_BK;
  const int rows_per_expert = DUAL ? 2 * p.N : p.N;

  if (warp == 0 && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
  }
  if (warp == 1 && lane == 0) {
    for (int s = 0; s < NSTAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(MG_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  pdl_wait();  // the offsets and the grouped rows come from the preceding kernels

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      TileCursor cur(p.offsets, p.n_experts, n_tiles_n, p.group_rows);
      int e, m0, m_end, n_blk;
      for (int tile = blockIdx.x; cur.seek(tile, e, m0, m_end, n_blk); tile += gridDim.x) {
        const int w_row = e * rows_per_expert + n_blk * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait_lim(empty_bar(stage), phase ^ 1, fail)) goto producer_done;
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          if (p.group_rows > 0) tma_load_2d(sa, &map_a, full_bar(stage), e * p.a_gs + kb * MG_BK, m0 - e * p.group_rows);
          else tma_load_2d(sa, &map_a, full_bar(stage), kb * MG_BK, m0);
          tma_load_2d(sa + MG_A_BYTES, &map_w, full_bar(stage), kb * MG_BK, w_row);
          if (DUAL) tma_load_2d(sa + MG_A_BYTES + W_BYTES, &map_w, full_bar(stage), kb * MG_BK, w_row + p.N);
          if (++stage == NSTAGES) { stage = 0; phase ^= 1; }
        }
      }
    producer_done:;
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      TileCursor cur(p.offsets, p.n_experts, n_tiles_n, p.group_rows);
      int e, m0, m_end, n_blk;
      for (int tile = blockIdx.x; cur.seek(tile, e, m0, m_end, n_blk); tile += gridDim.x) {
        if (!mbar_wait_lim(tempty_bar(acc), acc_phase ^ 1, fail)) goto mma_done;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait_lim(full_bar(stage), phase, fail)) goto mma_done;
          tc_fence_after();
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < MG_BK / MG_UMMA_K; ++k) {
            const uint64_t ad = umma_desc(sa + k * MG_UMMA_K * 2);
            const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
            umma(d_tmem, ad, umma_desc(sa + MG_A_BYTES + k * MG_UMMA_K * 2), IDESC, accumulate);
            if (DUAL) umma(d_tmem + BN, ad, umma_desc(sa + MG_A_BYTES + W_BYTES + k * MG_UMMA_K * 2), IDESC, accumulate);
          }
          umma_commit(empty_bar(stage));
          if (++stage == NSTAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit(tfull_bar(acc));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    mma_done:;
    }
  } else if (warp >= 4) {
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    T* out = reinterpret_cast<T*>(p.out);
    TileCursor cur(p.offsets, p.n_experts, n_tiles_n, p.group_rows);
    int e, m0, m_end, n_blk;
    for (int tile = blockIdx.x; cur.seek(tile, e, m0, m_end, n_blk); tile += gridDim.x) {
      if (!mbar_wait_lim(tfull_bar(acc), acc_phase, fail)) break;
      tc_fence_after();
      const int m = m0 + q * 32 + lane;
      // where this thread's row goes: the grouped row itself, or (per-head mode) its token row at the head's columns
      const size_t o_at = p.group_rows > 0 ? (size_t)(m - e * p.group_rows) * p.ldo + (size_t)e * p.o_gs : (size_t)m * p.ldo;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * ACC_COLS;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        float v[32], u[DUAL ? 32 : 1];
        tmem_ld32(t_row + c * 32, v);
        if (DUAL) tmem_ld32(t_row + BN + c * 32, u);
        tmem_ld_wait();
        const int n0 = n_blk * BN + c * 32;
        if (m < m_end && n0 < p.N) {
#pragma unroll
          for (int j0 = 0; j0 < 32; j0 += 8) {
            if (n0 + j0 >= p.N) break;  // N is a multiple of 8 (checked on the host)
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float x = rnd<T>(v[j0 + j]);
              if (DUAL) {
                float uu = rnd<T>(u[DUAL ? j0 + j : 0]);
                if (p.act == PG_GLU_CLAMPED) {
                  x = fminf(x, p.limit);
                  uu = fminf(fmaxf(uu, -p.limit), p.limit);
                  x = rnd<T>(x / (1.f + __expf(-1.702f * x))) * (uu + 1.f);
                } else {
                  x = rnd<T>(rnd<T>(x / (1.f + __expf(-x))) * uu);
                }
              }
              o[j] = x;
            }
            *reinterpret_cast<uint4*>(out + o_at + n0 + j0) = pack<T>(o);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (s_fail) {  // let copies and MMAs that are still in flight finish before the shared memory and TMEM go away
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && p.err_flag) *p.err_flag = 2;
    __syncthreads();
  }
  if (warp == 2) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(MG_TMEM_COLS) : "memory");
  }
}

template <typename T, bool DUAL, int BN>
static int launch_moe(const CUtensorMap& ma, const CUtensorMap& mw, const MoeParams& p, int max_tiles, cudaStream_t st) {
  constexpr int NSTAGES = (DUAL && BN > 64) ? 4 : 6;
  constexpr int STAGE_BYTES = MG_A_BYTES + (DUAL ? 2 : 1) * BN * MG_BK * 2;
  const size_t smem = 1024 + (size_t)NSTAGES * STAGE_BYTES + 8 * (2 * NSTAGES + 4) + 16;
  auto kern = moe_gemm_tc_kernel<T, DUAL, BN>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    set_error("moe_gemm_tc: cannot reserve %zu B of shared memory", smem);
    cudaGetLastError();
    return PG_ERR_CUDA;
  }
  return launch_tc("moe_gemm_tcgen05", kern, dim3(max_tiles < 148 ? max_tiles : 148), dim3(MG_THREADS), smem, 1, false, st,
                   ma, mw, p);
}

}  // namespace tc

bool moe_gemm_tc_supported(int ldo, int lda, const int32_t* row_map, int N, int K, int dtype) {
  static const int enabled = env_int("PG_MOE_TC", 1);
  if (!enabled || (dtype != PG_BF16 && dtype != PG_F16) || row_map != nullptr) return false;
  if (N % 8 || K % 8 || lda % 8 || ldo % 8) return false;
  return tc::encode_fn() != nullptr;
}

int moe_gemm_tc(void* out, int ldo, const void* A, int lda, const int32_t* row_map, const void* W,
                const int32_t* offsets, int n_pairs, int n_experts, int N, int K, int act, float limit, int dtype,
                int* err_flag, cudaStream_t st) {
  const int swiglu = act != PG_GLU_NONE;
  (void)row_map;
  PG_REQUIRE(((uintptr_t)A % 16) == 0 && ((uintptr_t)W % 16) == 0 && ((uintptr_t)out % 16) == 0,
             "moe_gemm_tc: operands must be 16-byte aligned");
  const bool bf = dtype == PG_BF16;
  const int bn = N >= 128 ? 128 : 64;
  const int rows_per_expert = swiglu ? 2 * N : N;
  CUtensorMap ma, mw;
  PG_REQUIRE(tc::make_map_2d(&ma, A, n_pairs, K, lda, tc::MG_BM, bf) &&
                 tc::make_map_2d(&mw, W, (long long)n_experts * rows_per_expert, K, K, bn, bf),
             "moe_gemm_tc: cuTensorMapEncodeTiled failed (rows=%d N=%d K=%d)", n_pairs, N, K);
  tc::MoeParams p = {out, offsets, n_experts, N, K, ldo, err_flag, act, limit, 0, 0, 0};
  const int max_tiles = (cdiv(n_pairs, tc::MG_BM) + n_experts) * cdiv(N, bn);
#define PG_MOE(D, B) return bf ? tc::launch_moe<bf16, D, B>(ma, mw, p, max_tiles, st) : tc::launch_moe<f16, D, B>(ma, mw, p, max_tiles, st)
  if (swiglu) { if (bn == 128) { PG_MOE(true, 128); } PG_MOE(true, 64); }
  if (bn == 128) { PG_MOE(false, 128); }
  PG_MOE(false, 64);
#undef PG_MOE
}

// Per-head products on token rows: out[t, h * o_gs + n] = sum_k A[t, h * a_gs + k] W[h][n][k] for all heads in ONE launch
// of the grouped kernel (a group = a head, every group the same n_rows token rows).
bool head_gemm_tc_supported(int ldo, int o_gs, int lda, int a_gs, int N, int K, int dtype) {
  static const int enabled = env_int("PG_HEAD_GEMM_TC", 1);
  if (!enabled || (dtype != PG_BF16 && dtype != PG_F16)) return false;
  if (N % 8 || K % 8 || lda % 8 || ldo % 8 || a_gs % 8 || o_gs % 8) return false;
  return tc::encode_fn() != nullptr;
}

int head_gemm_tc(void* out, int ldo, int o_gs, const void* A, int lda, int a_gs, const void* W, int n_rows, int heads, int N,
                 int K, int dtype, int* err_flag, cudaStream_t st) {
  PG_REQUIRE(((uintptr_t)A % 16) == 0 && ((uintptr_t)W % 16) == 0 && ((uintptr_t)out % 16) == 0,
             "head_gemm_tc: operands must be 16-byte aligned");
  const bool bf = dtype == PG_BF16;
  const int bn = N >= 128 ? 128 : 64;
  CUtensorMap ma, mw;
  PG_REQUIRE(tc::make_map_2d(&ma, A, n_rows, lda, lda, tc::MG_BM, bf) &&
                 tc::make_map_2d(&mw, W, (long long)heads * N, K, K, bn, bf),
             "head_gemm_tc: cuTensorMapEncodeTiled failed (rows=%d N=%d K=%d)", n_rows, N, K);
  tc::MoeParams p = {out, nullptr, heads, N, K, ldo, err_flag, PG_GLU_NONE, 0.f, n_rows, a_gs, o_gs};
  const int max_tiles = heads * cdiv(n_rows, tc::MG_BM) * cdiv(N, bn);
  if (bn == 128) return bf ? tc::launch_moe<bf16, false, 128>(ma, mw, p, max_tiles, st) : tc::launch_moe<f16, false, 128>(ma, mw, p, max_tiles, st);
  return bf ? tc::launch_moe<bf16, false, 64>(ma, mw, p, max_tiles, st) : tc::launch_moe<f16, false, 64>(ma, mw, p, max_tiles, st);
}

}  // namespace pg
