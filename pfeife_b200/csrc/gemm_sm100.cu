// Persistent warp-specialised GEMM for sm_100a: TMA -> 128B-swizzled smem ring -> tcgen05.mma
// with fp32 accumulators in TMEM (double buffered so the epilogue of tile i overlaps the main
// loop of tile i+1) -> tcgen05.ld -> fused epilogue -> global.
//
//   C[M,N] = epilogue(alpha * A[M,K] . B[N,K]^T)
//
// Each operand may be K-major (reduction index contiguous in memory) or MN-major (the M or N
// index contiguous); that covers forward (A K-major, B K-major), dgrad (A K-major, B MN-major)
// and wgrad (both MN-major) of a linear layer without a transpose pass.
//
// Epilogue (all optional, applied in this order): + bias[n], activation (GELU, saving the
// pre-activation to `aux`), multiply by gelu'(aux) (dGELU), + residual[m,n], accumulate into C
// (fp32 gradient buckets), cast to the output dtype.
//
// Role layout of the 320-thread CTA: warp 0 = TMA producer (one lane), warp 1 = TMEM owner and
// MMA issuer (one lane), warps 2..9 = epilogue (one accumulator row per thread; two warps share a
// TMEM lane quadrant and split the tile's columns, which halves the epilogue latency per tile);
// the instantiation that fuses an all-gather of B adds two warps that copy the remote rows.
#include <cstring>
#include "common.cuh"
#include "api.h"

namespace pf {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;       // 64 x 16-bit = one 128 B swizzle row
constexpr int GEMM_UMMA_K = 16;
constexpr int GEMM_EPI_WARPS = 8;     // two warps per TMEM lane quadrant, half the columns each
constexpr int GEMM_GATHER_WARPS = 2;  // copy remote rows of a sharded B operand (fused all-gather)
// the gather warps exist only in the instantiation that fuses the all-gather; without them the
// other roles may use more registers per thread
constexpr int gemm_threads(bool gather) {
  return 64 + 32 * (GEMM_EPI_WARPS + (gather ? GEMM_GATHER_WARPS : 0));
}

enum Epi : int { EPI_NONE = 0, EPI_GELU = 1, EPI_DGELU = 2, EPI_GELU_TANH = 3, EPI_DGELU_TANH = 4,
                 EPI_SILU = 5 };

struct GemmParams {
  int M, N, K;
  void* C;
  long long ldc;
  const void* bias;
  int bias_dtype;
  const void* residual;
  long long ldr;
  void* aux;
  long long ldaux;
  int epilogue;
  int accumulate;
  int vec_ok;     // C / residual / aux rows are 16-byte aligned at every 32-column chunk
  int tma_store;  // outputs leave through smem staging + TMA stores (needs vec_ok)
  float alpha;
  int a_mn, b_mn;
  int fmt;        // 0 = fp16 inputs, 1 = bf16 inputs
  int* status;
  int split_k;    // > 1: each tile's k-blocks are divided among this many work items, which all
                  // add into C (needs accumulate through the TMA reduce-add epilogue)
  // ---- fused all-gather of the B operand (weights sharded by rows over `gather_world` ranks)
  int gather_world;            // 0: B is an ordinary local operand
  int gather_rank;
  int gather_row_end[8];       // rank r owns rows [gather_row_end[r-1], gather_row_end[r]) of B
  const void* gather_src[8];   // every rank's copy of B [N, K] (pitch ldb), peer-mapped; only
                               // the rows a rank owns are valid (and read) in its copy
  void* gather_dst;            // local full-size B [N, K] (pitch ldb); own rows already in place
  int* gather_ready;           // local counters, one per BN-row tile of B, zeroed before launch
  long long gather_ld;
  // ---- implicit-GEMM convolution: A is an NHWC activation [B, H, W, C] read through a 4-D
  //      tensor map; row m of the GEMM is output pixel m (tiles of 128 rows = whole output rows
  //      of one image), k-block kb is filter tap (r, s) = kb / (C/64) and channels
  //      64 * (kb % (C/64)); padding comes from the TMA out-of-bounds fill
  //      conv == 2 (weight gradient): B is the activation instead, read as an MN-major operand:
  //      k-block kb is 64 consecutive output pixels, column n of the GEMM is filter tap n / C
  //      and channel n % C
  int conv;                    // 0: plain matrices, 1: A from the activation, 2: B from it
  int conv_c64;                // C / 64
  int conv_kw, conv_pad, conv_stride;
  int conv_wo, conv_howo;      // output width, output pixels per image
};

template <int BN, int STAGES, int SPW>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  // epilogue staging for TMA stores: SPW bytes per epilogue warp, holding [32 rows x 32 cols]
  // boxes (2 KB for 16-bit outputs, 4 KB for fp32): C and, when saved, aux; twice over when
  // SPW has room for it
  static constexpr int STAGING_OFFSET = BAR_OFFSET + 1024;
  static constexpr int STAGING_PER_WARP = SPW;
  static constexpr int TOTAL = STAGING_OFFSET + GEMM_EPI_WARPS * STAGING_PER_WARP + 1024;
};

__device__ __forceinline__ float load_bias(const void* bias, int dtype, int n) {
  if (dtype == PF_F32) return __ldg(reinterpret_cast<const float*>(bias) + n);
  if (dtype == PF_F16) return __half2float(__ldg(reinterpret_cast<const __half*>(bias) + n));
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias)[n]);
}

template <typename OutT>
__device__ __forceinline__ void load_row32(const OutT* p, bool vec, int nvalid, float (&v)[32]) {
  if (vec && nvalid == 32) {
    constexpr int PER = 16 / sizeof(OutT);
    constexpr int NV = 32 / PER;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      uint4 q = __ldg(reinterpret_cast<const uint4*>(p) + i);
      const OutT* e = reinterpret_cast<const OutT*>(&q);
#pragma unroll
      for (int j = 0; j < PER; ++j) v[i * PER + j] = to_f32<OutT>(e[j]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = (i < nvalid) ? to_f32<OutT>(p[i]) : 0.f;
  }
}

template <typename OutT>
__device__ __forceinline__ void store_row32(OutT* p, bool vec, int nvalid, const float (&v)[32]) {
  if (vec && nvalid == 32) {
    constexpr int PER = 16 / sizeof(OutT);
    constexpr int NV = 32 / PER;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      uint4 q;
      OutT* e = reinterpret_cast<OutT*>(&q);
#pragma unroll
      for (int j = 0; j < PER; ++j) e[j] = from_f32<OutT>(v[i * PER + j]);
      reinterpret_cast<uint4*>(p)[i] = q;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < nvalid) p[i] = from_f32<OutT>(v[i]);
  }
}

// Writes row `r` (32 values) of a [32 x 32] staging box in the swizzled layout the TMA store
// expects: 64-byte rows with SWIZZLE_64B for 16-bit outputs, 128-byte rows with SWIZZLE_128B
// for fp32 outputs.  Conflict-free across the 32 lanes of a warp.
template <typename OutT>
__device__ __forceinline__ void stage_row32(uint8_t* box, int r, const float (&v)[32]) {
  constexpr int PER = 16 / sizeof(OutT);
  constexpr int NCH = 32 / PER;            // 4 (16-bit) or 8 (fp32) 16-byte chunks per row
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    uint4 q;
    OutT* e = reinterpret_cast<OutT*>(&q);
#pragma unroll
    for (int j = 0; j < PER; ++j) e[j] = from_f32<OutT>(v[c * PER + j]);
    const int sw = (NCH == 4) ? (c ^ ((r >> 1) & 3)) : (c ^ (r & 7));
    *reinterpret_cast<uint4*>(box + r * (NCH * 16) + sw * 16) = q;
  }
}

// PAIR = false: one CTA per 128 x BN tile.  PAIR = true: the kernel runs as clusters of two CTAs
// that share one 256 x 2BN tile through tcgen05.mma.cta_group::2: each CTA loads 128 rows of A
// and BN rows of B per k-block (half the shared-memory traffic per FLOP of the single-CTA form),
// the even CTA issues the MMAs, and each CTA's TMEM receives -- and its epilogue warps drain --
// the 128 accumulator rows that match its rows of A.
template <typename OutT, int BN, int STAGES, int SPW, bool PAIR, bool GATHER>
__global__ void __launch_bounds__(gemm_threads(GATHER), 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                    const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_c,
                    const __grid_constant__ CUtensorMap tmap_aux, const GemmParams p) {
  using S = GemmSmem<BN, STAGES, SPW>;
  extern __shared__ uint8_t smem_raw[];
  // 128B swizzle atoms need 1024 B alignment
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int BNT = PAIR ? 2 * BN : BN;          // columns of the output tile
  constexpr int BMT = PAIR ? 2 * GEMM_BM : GEMM_BM; // rows of the output tile (both CTAs of a pair)
  constexpr uint32_t TMEM_COLS = 2 * BNT;  // 256 or 512: a power of two
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
  const int first_tile = PAIR ? (blockIdx.x >> 1) : blockIdx.x;
  const int tile_step = PAIR ? (gridDim.x >> 1) : gridDim.x;

  const int num_m = (p.M + BMT - 1) / BMT;
  const int num_n = (p.N + BNT - 1) / BNT;
  const int split_k = p.split_k > 1 ? p.split_k : 1;
  const int num_tiles = num_m * num_n * split_k;        // work items: (tile, k-slice)
  const int num_kb = (p.K + GEMM_BK - 1) / GEMM_BK;
  const int num_mn = num_m * num_n;
  // Work items are dealt to the CTAs (pairs) in rounds, every other round in reverse order.
  // Items are ordered with the cheap ones last (the tiles of a narrow last column of tiles),
  // so the CTAs that got an expensive item late in one round get a cheap one in the next.
  const int n_workers = tile_step;
  auto item_of = [&](int round) -> int {
    const int slot = (round & 1) ? (n_workers - 1 - first_tile) : first_tile;
    return round * n_workers + slot;
  };
  // pair tiles in the last column of tiles run a narrower MMA when at most half of their
  // columns exist: each CTA then supplies 64 rows of B instead of 128
  const int edge_cols = p.N - (num_n - 1) * BNT;
  const bool narrow_edge = PAIR && BNT == 256 && edge_cols <= 128;
  // with a fused all-gather the tiles whose rows of B this rank owns are computed first, while
  // the remote rows are still arriving
  const int own0 = (GATHER && p.gather_rank > 0) ? p.gather_row_end[p.gather_rank - 1] : 0;
  const int own1 = GATHER ? p.gather_row_end[p.gather_rank] : 0;
  const int n_rot = (GATHER && p.gather_world > 1) ? own0 / BNT : 0;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      // single CTA: every epilogue thread arrives; pair: lane 0 of every epilogue warp of both
      // CTAs arrives on the leader's barrier
      mbar_init(&tmem_empty[i], PAIR ? 2 * GEMM_EPI_WARPS : 32 * GEMM_EPI_WARPS);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(tmem_slot, TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync();   // the peer's barriers exist before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      bool all_gathered = false;
      // pair: both CTAs' loads of a stage are counted on the leader's barrier
      for (int round = 0, item = item_of(0); item < num_tiles && ok; item = item_of(++round)) {
        const int tile = item % num_mn, ks = item / num_mn;
        const int kb_begin = (int)((long long)num_kb * ks / split_k);
        const int kb_end = (int)((long long)num_kb * (ks + 1) / split_k);
        const int m0 = (tile % num_m) * BMT + int(cta_rank) * GEMM_BM;
        const int nt = (tile / num_m + n_rot) % num_n;
        const int n0 = nt * BNT;
        // first row of B this CTA loads: its half of the columns the MMA computes
        const int nb0 = n0 + int(cta_rank) * ((narrow_edge && nt == num_n - 1) ? BN / 2 : BN);
        if (GATHER && p.gather_world > 1 && !all_gathered) {
          // rows of this B tile that other ranks own must have landed in the local buffer
          const int n1 = min(p.N, n0 + BNT);
          const int expect = (n1 - n0) - max(0, min(n1, own1) - max(n0, own0));
          if (expect > 0) {
            const long long t0 = clock64(), limit = wait_limit(p.status);
            while (*reinterpret_cast<volatile int*>(p.gather_ready + nt) < expect) {
              if (clock64() - t0 > limit) { report(p.status, PF_ERR_TIMEOUT_PEER_FLAG); ok = false; break; }
            }
            // once every remote row is in place no later tile needs to look again
            const int remote_rows = p.N - max(0, min(p.N, own1) - own0);
            all_gathered = *reinterpret_cast<volatile int*>(p.gather_ready + num_n) >= remote_rows;
            __threadfence();
            asm volatile("fence.proxy.async;" ::: "memory");   // generic writes -> TMA reads
            if (!ok) break;
          }
        }
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, p.status, PF_ERR_TIMEOUT_EMPTY);
          if (!ok) break;
          uint8_t* sa = smem + stage * S::STAGE_BYTES;
          uint8_t* sb = sa + S::A_BYTES;
          const int k0 = kb * GEMM_BK;
          // implicit-GEMM convolution: coordinates of this k-block's 128-pixel window
          int cv_c = 0, cv_w = 0, cv_h = 0, cv_b = 0;
          if (p.conv == 2) {     // the 64 output pixels of this k-block (part of one image)
            const int p0 = kb * GEMM_BK;
            cv_b = p0 / p.conv_howo;
            const int rem = p0 - cv_b * p.conv_howo;
            cv_h = (rem / p.conv_wo) * p.conv_stride - p.conv_pad;
            cv_w = (rem % p.conv_wo) * p.conv_stride - p.conv_pad;
          } else if (p.conv) {
            const int tap = kb / p.conv_c64;
            cv_c = (kb - tap * p.conv_c64) * 64;
            const int r = tap / p.conv_kw, sx = tap - r * p.conv_kw;
            cv_b = m0 / p.conv_howo;
            const int ho0 = (m0 - cv_b * p.conv_howo) / p.conv_wo;
            cv_w = sx - p.conv_pad;
            cv_h = ho0 * p.conv_stride + r - p.conv_pad;
          }
          if (PAIR) {
            if (cta_rank == 0) mbar_expect_tx(&full_bar[stage], 2 * S::STAGE_BYTES);
            const uint32_t bar = mapa_u32(&full_bar[stage], 0);
            if (p.conv == 1) {
              tma_load_4d_pair(sa, &tmap_a, bar, cv_c, cv_w, cv_h, cv_b);
            } else if (!p.a_mn) {
              tma_load_2d_pair(sa, &tmap_a, bar, k0, m0);
            } else {
#pragma unroll
              for (int j = 0; j < GEMM_BM / 64; ++j)
                tma_load_2d_pair(sa + j * 8192, &tmap_a, bar, m0 + j * 64, k0);
            }
            if (p.conv == 2) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) {
                const int n = nb0 + j * 64, tap = n / (p.conv_c64 * 64);
                const int r = tap / p.conv_kw, sx = tap - r * p.conv_kw;
                tma_load_4d_pair(sb + j * 8192, &tmap_b, bar, n - tap * p.conv_c64 * 64,
                                 cv_w + sx, cv_h + r, cv_b);
              }
            } else if (!p.b_mn) {
              tma_load_2d_pair(sb, &tmap_b, bar, k0, nb0);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d_pair(sb + j * 8192, &tmap_b, bar, nb0 + j * 64, k0);
            }
          } else {
            mbar_expect_tx(&full_bar[stage], S::STAGE_BYTES);
            if (p.conv == 1) {
              tma_load_4d(sa, &tmap_a, &full_bar[stage], cv_c, cv_w, cv_h, cv_b);
            } else if (!p.a_mn) {
              tma_load_2d(sa, &tmap_a, &full_bar[stage], k0, m0);
            } else {
#pragma unroll
              for (int j = 0; j < GEMM_BM / 64; ++j)
                tma_load_2d(sa + j * 8192, &tmap_a, &full_bar[stage], m0 + j * 64, k0);
            }
            if (p.conv == 2) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) {
                const int n = n0 + j * 64, tap = n / (p.conv_c64 * 64);
                const int r = tap / p.conv_kw, sx = tap - r * p.conv_kw;
                tma_load_4d(sb + j * 8192, &tmap_b, &full_bar[stage], n - tap * p.conv_c64 * 64,
                            cv_w + sx, cv_h + r, cv_b);
              }
            } else if (!p.b_mn) {
              tma_load_2d(sb, &tmap_b, &full_bar[stage], k0, n0);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(sb + j * 8192, &tmap_b, &full_bar[stage], n0 + j * 64, k0);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && cta_rank == 0) {
      const uint32_t idesc = make_idesc_f16(BMT, BNT, p.fmt, p.a_mn, p.b_mn);
      // per-UMMA_K advance of the descriptor start address and its LBO/SBO
      const uint32_t a_adv = p.a_mn ? 2048u : 32u;
      const uint32_t b_adv = p.b_mn ? 2048u : 32u;
      const uint32_t a_lbo = p.a_mn ? 8192u : 16u;
      const uint32_t b_lbo = p.b_mn ? 8192u : 16u;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      const uint32_t idesc_narrow = make_idesc_f16(BMT, BNT / 2, p.fmt, p.a_mn, p.b_mn);
      for (int round = 0, item = item_of(0); item < num_tiles && ok; item = item_of(++round)) {
        const int ks = item / num_mn;
        const int kb_begin = (int)((long long)num_kb * ks / split_k);
        const int kb_end = (int)((long long)num_kb * (ks + 1) / split_k);
        const bool narrow = narrow_edge && ((item % num_mn) / num_m + n_rot) % num_n == num_n - 1;
        const uint32_t idesc_t = narrow ? idesc_narrow : idesc;
        ok = PAIR ? mbar_wait_cluster(&tmem_empty[acc], acc_phase ^ 1, p.status,
                                      PF_ERR_TIMEOUT_TMEM_EMPTY)
                  : mbar_wait(&tmem_empty[acc], acc_phase ^ 1, p.status,
                              PF_ERR_TIMEOUT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BNT;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, p.status, PF_ERR_TIMEOUT_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < GEMM_BK / GEMM_UMMA_K; ++k) {
            const uint64_t da = make_desc_sw128(sa + k * a_adv, a_lbo, 1024);
            const uint64_t db = make_desc_sw128(sb + k * b_adv, b_lbo, 1024);
            const uint32_t acc_on = (kb != kb_begin) || (k != 0);
            if (PAIR) tc_mma_f16_pair(d_tmem, da, db, idesc_t, acc_on);
            else tc_mma_f16(d_tmem, da, db, idesc_t, acc_on);
          }
          // smem slot reusable (in both CTAs of a pair) once these MMAs retire
          if (PAIR) tc_commit_pair(&empty_bar[stage], 3);
          else tc_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (PAIR) tc_commit_pair(&tmem_full[acc], 3);
        else tc_commit(&tmem_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
    __syncwarp();
  } else if (warp >= 2 + GEMM_EPI_WARPS) {
    // ------------------------------------------------------------------ gather warps
    if (GATHER && p.gather_world > 1) {
      // All-gather of the remote shards of B: the gather warps of every CTA copy whole
      // rows from the owners' memory (plain peer loads, 16 bytes per lane) into the local
      // buffer and bumps the counter of the row's tile.  The TMA producer of a tile waits for
      // its counter, so the transfer overlaps the tiles computed before it.
      const int ew = blockIdx.x * GEMM_GATHER_WARPS + (warp - 2 - GEMM_EPI_WARPS);
      const int n_ew = gridDim.x * GEMM_GATHER_WARPS;
      const int kvec = p.K / 8;
      for (int r = ew; r < p.N; r += n_ew) {
        if (r >= own0 && r < own1) continue;
        int owner = 0;
        while (owner < p.gather_world - 1 && r >= p.gather_row_end[owner]) ++owner;
        const uint4* src = reinterpret_cast<const uint4*>(
            reinterpret_cast<const uint16_t*>(p.gather_src[owner]) + (long long)r * p.gather_ld);
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.gather_dst) +
                                              (long long)r * p.gather_ld);
        // up to 8 vectors per lane are requested before any is stored (latency hiding)
        for (int c0 = lane; c0 < kvec; c0 += 256) {
          uint4 buf[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (c0 + u * 32 < kvec) buf[u] = src[c0 + u * 32];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (c0 + u * 32 < kvec) dst[c0 + u * 32] = buf[u];
        }
        asm volatile("fence.proxy.async;" ::: "memory");
        __threadfence();
        __syncwarp();
        if (lane == 0) {
          atomicAdd(p.gather_ready + r / BNT, 1);
          atomicAdd(p.gather_ready + num_n, 1);   // running total of gathered rows
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (8 warps)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const int col_half = (warp - 2) >> 2;          // which half of the tile's columns
    const int c_begin = col_half * (BNT / 2), c_end = c_begin + BNT / 2;
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    OutT* C = reinterpret_cast<OutT*>(p.C);
    const OutT* R = reinterpret_cast<const OutT*>(p.residual);
    OutT* AUX = reinterpret_cast<OutT*>(p.aux);
    const bool aux_out = AUX && (p.epilogue == EPI_GELU || p.epilogue == EPI_GELU_TANH ||
                                 p.epilogue == EPI_SILU);
    // Staging for TMA stores: a set is the C box (2 KB for 16-bit outputs, 4 KB for fp32) plus,
    // when the pre-activation is saved, the aux box.  With room for two sets the warp fills one
    // while the stores of the other are still reading it.
    uint8_t* stage_base = smem + S::STAGING_OFFSET + (warp - 2) * S::STAGING_PER_WARP;
    const int set_bytes = (sizeof(OutT) == 4 || aux_out) ? 4096 : 2048;
    const bool two_sets = S::STAGING_PER_WARP >= 2 * set_bytes;
    int set = 0;
    int staged = 0;        // chunks handed to the TMA so far (saturates at 2)
    const bool vec = p.vec_ok != 0;
    const bool tma_out = p.tma_store != 0;
    const bool bias_vec = p.bias && p.bias_dtype == PF_F32 &&
                          (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0;
    for (int round = 0, item = item_of(0); item < num_tiles && ok; item = item_of(++round)) {
      const int tile = item % num_mn;
      const int m0 = (tile % num_m) * BMT + int(cta_rank) * GEMM_BM;
      const int n0 = ((tile / num_m + n_rot) % num_n) * BNT;
      ok = mbar_wait(&tmem_full[acc], acc_phase, p.status, PF_ERR_TIMEOUT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + row_in_tile;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + (uint32_t(quad * 32) << 16) + acc * BNT;
      uint32_t raw[32];
      if (n0 + c_begin < p.N) tmem_ld32(t_row + c_begin, raw);   // uniform across the warp
#pragma unroll 1
      for (int c = c_begin; c < c_end; c += 32) {
        const int col = n0 + c;
        if (col >= p.N) break;  // uniform across the warp
        tmem_ld_wait_for(raw);
        const int nvalid = min(32, p.N - col);
        float v[32];
        if (p.alpha != 1.0f) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]) * p.alpha;
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]);
        }
        // the next chunk's accumulators travel from TMEM while this one is processed
        if (c + 32 < c_end && col + 32 < p.N) tmem_ld32(t_row + c + 32, raw);
        if (p.bias) {
          if (bias_vec && nvalid == 32) {
            const float4* bp = reinterpret_cast<const float4*>(
                reinterpret_cast<const float*>(p.bias) + col);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 b4 = __ldg(bp + j);
              v[4 * j] += b4.x; v[4 * j + 1] += b4.y; v[4 * j + 2] += b4.z; v[4 * j + 3] += b4.w;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < nvalid) v[i] += load_bias(p.bias, p.bias_dtype, col + i);
          }
        }
        uint8_t* stage_c = stage_base + set * set_bytes;
        uint8_t* stage_aux = stage_c + 2048;           // only used by 16-bit outputs
        if (tma_out && staged >= (two_sets ? 2 : 1)) {
          // the stores that last used this set must have read it before it is refilled
          if (lane == 0) {
            if (two_sets) tma_store_wait_read_but_one();
            else tma_store_wait_read();
          }
          __syncwarp();
        }
        if (p.epilogue == EPI_GELU || p.epilogue == EPI_GELU_TANH || p.epilogue == EPI_SILU) {
          if (aux_out) {
            if (tma_out) stage_row32<OutT>(stage_aux, lane, v);
            else if (row_ok)
              store_row32<OutT>(AUX + (long long)row * p.ldaux + col, vec, nvalid, v);
          }
          if (p.epilogue == EPI_GELU) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = gelu_erf_fast(v[i]);
          } else if (p.epilogue == EPI_GELU_TANH) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(v[i]);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = silu(v[i]);
          }
        } else if ((p.epilogue == EPI_DGELU || p.epilogue == EPI_DGELU_TANH) && row_ok) {
          float z[32];
          load_row32<OutT>(AUX + (long long)row * p.ldaux + col, vec, nvalid, z);
          if (p.epilogue == EPI_DGELU) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= dgelu_erf_fast(z[i]);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= dgelu_tanh(z[i]);
          }
        }
        if (R && row_ok) {
          float r[32];
          load_row32<OutT>(R + (long long)row * p.ldr + col, vec, nvalid, r);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] += r[i];
        }
        if (tma_out) {
          // rows / columns beyond M / N are clipped by the TMA store itself
          stage_row32<OutT>(stage_c, lane, v);
          fence_async_smem();
          __syncwarp();
          const int row0 = m0 + quad * 32;
          if (lane == 0 && row0 < p.M) {
            if (p.accumulate) tma_reduce_add_2d(&tmap_c, stage_c, col, row0);
            else tma_store_2d(&tmap_c, stage_c, col, row0);
            if (aux_out) tma_store_2d(&tmap_aux, stage_aux, col, row0);
          }
          // an (empty) group is committed even for a clipped chunk so that the group count
          // matches the set rotation
          if (lane == 0) tma_store_commit();
          if (staged < 2) ++staged;
          if (two_sets) set ^= 1;
        } else if (row_ok) {
          OutT* dst = C + (long long)row * p.ldc + col;
          if (p.accumulate) {
            float o[32];
            load_row32<OutT>(dst, vec, nvalid, o);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] += o[i];
          }
          store_row32<OutT>(dst, vec, nvalid, v);
        }
      }
      tc_fence_before();
      if (PAIR) {
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_u32(&tmem_empty[acc], 0));
      } else {
        mbar_arrive(&tmem_empty[acc]);
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  // teardown: every role reaches this point (all waits are bounded)
  if (warp >= 2 && lane == 0 && p.tma_store) tma_store_wait_all();
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync();   // neither CTA leaves while the other may still signal it
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D map over a row-major [outer, inner] 16-bit tensor with row pitch `ld` elements.
int make_tmap_2d_16bit(CUtensorMap* map, const void* base, int fmt, long long inner,
                       long long outer, long long ld, int box_inner, int box_outer) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -100;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, fmt ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                   2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(1000 + (int)r);
}

// [rows, cols] output map with a 32 x 32 box; 16-bit: 64 B rows (SWIZZLE_64B), fp32: 128 B rows
// (SWIZZLE_128B)
static int make_tmap_out(CUtensorMap* map, const void* base, int out_dtype, long long cols,
                         long long rows, long long ld) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -100;
  const int es = out_dtype == PF_F32 ? 4 : 2;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * es};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = out_dtype == PF_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : out_dtype == PF_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                        : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   out_dtype == PF_F32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(1000 + (int)r);
}

template <typename OutT, int BN, int STAGES, int SPW, bool PAIR, bool GATHER>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                       const CUtensorMap& taux, const GemmParams& p, int sm_count,
                       cudaStream_t stream) {
  using S = GemmSmem<BN, STAGES, SPW>;
  constexpr int THREADS = gemm_threads(GATHER);
  auto kern = gemm_tcgen05_kernel<OutT, BN, STAGES, SPW, PAIR, GATHER>;
  static bool configured[64] = {};  // the attribute is per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  if (PAIR) {
    const int num_tiles = ((p.M + 2 * GEMM_BM - 1) / (2 * GEMM_BM)) *
                          ((p.N + 2 * BN - 1) / (2 * BN)) * (p.split_k > 1 ? p.split_k : 1);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (sm_count / 2));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = S::TOTAL;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // pairs that can be resident at once (the two CTAs of a pair sit on neighbouring SMs)
    static int resident_pairs[64] = {};
    int max_pairs = (dev >= 0 && dev < 64) ? resident_pairs[dev] : 0;
    if (max_pairs == 0) {
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();
        n = sm_count / 2;
      }
      max_pairs = n < sm_count / 2 ? n : sm_count / 2;
      if (dev >= 0 && dev < 64) resident_pairs[dev] = max_pairs;
    }
    const int pairs = num_tiles < max_pairs ? num_tiles : max_pairs;
    cfg.gridDim = dim3(2 * pairs);
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, taux, p);
    if (e != cudaSuccess) return (int)e;
    return 0;
  }
  const int num_tiles = ((p.M + GEMM_BM - 1) / GEMM_BM) * ((p.N + BN - 1) / BN) *
                        (p.split_k > 1 ? p.split_k : 1);
  const int grid = num_tiles < sm_count ? num_tiles : sm_count;
  kern<<<grid, THREADS, S::TOTAL, stream>>>(ta, tb, tc, taux, p);
  PF_CHECK_LAUNCH();
  return 0;
}

}  // namespace pf

using namespace pf;

// 4-D map over an NHWC activation [B, H, W, C] (16-bit): box = 64 channels x `box_w` x `box_h`
// pixels of one image, traversed with `stride` in both spatial dimensions
static int make_tmap_nhwc(CUtensorMap* map, const void* base, int fmt, int B, int H, int W, int C,
                          int box_w, int box_h, int stride) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -100;
  cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)C * 2, (cuuint64_t)W * C * 2, (cuuint64_t)H * W * C * 2};
  // a box dimension is the extent it spans in the tensor: `stride` times the pixels it delivers
  cuuint32_t box[4] = {64, (cuuint32_t)(box_w * stride), (cuuint32_t)(box_h * stride), 1};
  cuuint32_t estr[4] = {1, (cuuint32_t)stride, (cuuint32_t)stride, 1};
  CUresult r = enc(map, fmt ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                   4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(1000 + (int)r);
}

// convolution geometry of the call in flight on this thread (set by pf_conv_gemm)
struct ConvArgs { int on = 0, B = 0, H = 0, W = 0, C = 0, KH = 0, KW = 0, stride = 1, pad = 0,
                  Ho = 0, Wo = 0; };
static thread_local ConvArgs g_conv;

// all-gather arguments of the call in flight on this thread (set by pf_gemm_allgather)
struct GatherArgs {
  int world = 0, rank = 0; int row_end[8] = {}; int* ready = nullptr; const void* src[8] = {};
  bool on_any() const { return world > 1; }
};
static thread_local GatherArgs g_gather;

PF_API int pf_gemm(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                   long long ldb, long long ldc, int a_mn, int b_mn, int in_dtype, int out_dtype,
                   const void* bias, int bias_dtype, const void* residual, long long ldr,
                   void* aux, long long ldaux, int epilogue, int accumulate, float alpha,
                   int* status, int sm_count, int tile_n, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (in_dtype != PF_F16 && in_dtype != PF_BF16) return -1;
  if ((g_conv.on != 1 && (lda % 8)) || (g_conv.on != 2 && (ldb % 8)) ||
      (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15))
    return -2;  // TMA needs 16-byte aligned bases and pitches
  const int fmt = in_dtype == PF_BF16 ? 1 : 0;
  // tile_n: low bits 0 / 128 / 256 = tile width of the single-CTA form; bit 10 forces the
  // direct-store epilogue, bit 11 forces the CTA-pair form, bit 12 forbids it, bit 13 forbids
  // the split reduction (tests, benches)
  const int tn = tile_n & 1023;
  if (sm_count <= 0) sm_count = 148;
  bool pair = false;
  if (g_gather.world <= 1 && !(tile_n & 4096) && sm_count >= 2) {
    if (tile_n & 2048) {
      pair = true;
    } else if (tn == 0 && M > 128 && N > 128) {
      // rounds of 256 x 256 pair tiles over sm_count / 2 pairs against rounds of 128 x 256 tiles
      // over sm_count CTAs.  Measured on B200, a pair tile costs each SM 0.9-0.95 of a single
      // tile when both fill their rounds, but more than a single tile on long-K shapes with a
      // narrow last column of tiles (N = 1408, K = 6144: 126 us against 107 us), so pairs are
      // taken only when 0.93 of their rounds is no more than the single-CTA rounds.
      const long long t2 = (long long)((M + 255) / 256) * ((N + 255) / 256);
      const long long t1 = (long long)((M + 127) / 128) * ((N + 255) / 256);
      const long long w2 = (t2 + sm_count / 2 - 1) / (sm_count / 2);
      const long long w1 = (t1 + sm_count - 1) / sm_count;
      pair = 93 * w2 <= 100 * w1;
    }
  }
  int bn_auto = N <= 128 ? 128 : 256;
  if (!pair && tn == 0 && N > 128) {
    // 128 x 128 tiles (0.55 of a 128 x 256 tile each) when they fill the waves better
    const long long t1 = (long long)((M + 127) / 128) * ((N + 255) / 256);
    const long long th = (long long)((M + 127) / 128) * ((N + 127) / 128);
    const long long w1 = (t1 + sm_count - 1) / sm_count;
    const long long wh = (th + sm_count - 1) / sm_count;
    if (11 * wh < 20 * w1) bn_auto = 128;
  }
  const int BN = pair ? 128 : (tn == 128 || tn == 256) ? tn : bn_auto;

  CUtensorMap ta, tb;
  int r;
  if (g_conv.on == 1)
    r = make_tmap_nhwc(&ta, A, fmt, g_conv.B, g_conv.H, g_conv.W, g_conv.C, g_conv.Wo,
                       GEMM_BM / g_conv.Wo, g_conv.stride);
  else if (!a_mn) r = make_tmap_2d_16bit(&ta, A, fmt, K, M, lda, GEMM_BK, GEMM_BM);
  else       r = make_tmap_2d_16bit(&ta, A, fmt, M, K, lda, 64, GEMM_BK);
  if (r) return r;
  if (g_conv.on == 2) {
    const int bw = g_conv.Wo < GEMM_BK ? g_conv.Wo : GEMM_BK;
    r = make_tmap_nhwc(&tb, B, fmt, g_conv.B, g_conv.H, g_conv.W, g_conv.C, bw, GEMM_BK / bw,
                       g_conv.stride);
  } else if (!b_mn) r = make_tmap_2d_16bit(&tb, B, fmt, K, N, ldb, GEMM_BK, BN);
  else       r = make_tmap_2d_16bit(&tb, B, fmt, N, K, ldb, 64, GEMM_BK);
  if (r) return r;

  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.bias = bias; p.bias_dtype = bias_dtype;
  p.residual = residual; p.ldr = ldr;
  p.aux = aux; p.ldaux = ldaux;
  p.epilogue = epilogue; p.accumulate = accumulate;
  p.alpha = alpha; p.a_mn = a_mn; p.b_mn = b_mn; p.fmt = fmt; p.status = status;
  p.gather_world = g_gather.world; p.gather_rank = g_gather.rank;
  for (int i = 0; i < 8; ++i) p.gather_row_end[i] = g_gather.row_end[i];
  p.gather_dst = const_cast<void*>(B);
  p.gather_ready = g_gather.ready; p.gather_ld = ldb;
  for (int i = 0; i < 8; ++i) p.gather_src[i] = g_gather.src[i];
  p.conv = g_conv.on;
  if (g_conv.on) {
    p.conv_c64 = g_conv.C / 64; p.conv_kw = g_conv.KW; p.conv_pad = g_conv.pad;
    p.conv_stride = g_conv.stride; p.conv_wo = g_conv.Wo; p.conv_howo = g_conv.Ho * g_conv.Wo;
  }
  const size_t es = out_dtype == PF_F32 ? 4 : 2;
  auto aligned = [&](const void* ptr, long long ld) {
    return ptr == nullptr || ((reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && (ld * es) % 16 == 0);
  };
  p.vec_ok = aligned(C, ldc) && aligned(residual, ldr) && aligned(aux, ldaux);
  // TMA-store epilogue: needs aligned outputs; fp32 accumulation uses the reduce-add store,
  // 16-bit accumulation (unused by the framework) stays on the direct path
  p.tma_store = p.vec_ok && !(accumulate && out_dtype != PF_F32) && !(tile_n & 1024) &&
                !(aux && out_dtype == PF_F32);
  // Split-K: a gradient-accumulating GEMM whose tiles do not fill the GPU divides each tile's
  // reduction among several work items; they all reduce-add into C, which costs nothing extra
  // because the epilogue accumulates anyway.
  p.split_k = 1;
  if (p.tma_store && accumulate && out_dtype == PF_F32 && !g_gather.on_any() && !g_conv.on &&
      !bias && !residual && epilogue == EPI_NONE && !(tile_n & 8192)) {
    const int bm = pair ? 256 : 128, bn = pair ? 256 : BN;
    const long long tiles = (long long)((M + bm - 1) / bm) * ((N + bn - 1) / bn);
    const long long slots = pair ? sm_count / 2 : sm_count;
    const int nkb = (K + GEMM_BK - 1) / GEMM_BK;
    double best = 1e30;
    for (int sk = 1; sk <= 4 && sk * 8 <= nkb; ++sk) {
      const double waves = (double)((tiles * sk + slots - 1) / slots) / sk + 0.03 * (sk - 1);
      if (waves < best - 1e-9) { best = waves; p.split_k = sk; }
    }
  }
  CUtensorMap tc, taux;
  memset(&tc, 0, sizeof(tc));
  memset(&taux, 0, sizeof(taux));
  if (p.tma_store) {
    if ((r = make_tmap_out(&tc, C, out_dtype, N, M, ldc))) return r;
    const bool aux_is_out = aux && (epilogue == EPI_GELU || epilogue == EPI_GELU_TANH ||
                                    epilogue == EPI_SILU);
    if (aux_is_out && (r = make_tmap_out(&taux, aux, out_dtype, N, M, ldaux))) return r;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

  const bool gather = g_gather.world > 1;
#define PF_GEMM_DISPATCH(T)                                                                    \
  (pair     ? launch_gemm<T, 128, 5, 8192, true, false>(ta, tb, tc, taux, p, sm_count, st)     \
   : gather ? launch_gemm<T, 256, 4, 4096, false, true>(ta, tb, tc, taux, p, sm_count, st)     \
   : BN == 256 ? launch_gemm<T, 256, 4, 4096, false, false>(ta, tb, tc, taux, p, sm_count, st) \
               : launch_gemm<T, 128, 5, 8192, false, false>(ta, tb, tc, taux, p, sm_count, st))
  switch (out_dtype) {
    case PF_F32: return PF_GEMM_DISPATCH(float);
    case PF_F16: return PF_GEMM_DISPATCH(__half);
    case PF_BF16: return PF_GEMM_DISPATCH(__nv_bfloat16);
  }
  return -1;
}

// C[M,N] = epi(A[M,K] . W[N,K]^T) where the rows of W are owned by `world` ranks: rank r owns
// rows [row_end[r-1], row_end[r]) (row_end[world-1] == N) and `copies[r]` points at rank r's
// full-size copy of W (pitch ldb, peer-mapped for r != rank) in which at least the rows it owns
// are current.  `w_full` is this rank's copy; the kernel fills in the other ranks' rows while it
// computes.  `ready` is an int array with one entry per 256-row tile of W plus one for the
// running total (zeroed here).
PF_API int pf_gemm_allgather(const void* A, void* w_full, void* const* copies, int world, int rank,
                             const int* row_end, void* ready, void* C, int M, int N, int K,
                             long long lda, long long ldb, long long ldc, int in_dtype,
                             int out_dtype, const void* bias, int bias_dtype,
                             const void* residual, long long ldr, void* aux, long long ldaux,
                             int epilogue, float alpha, int* status, int sm_count, void* stream) {
  if (world < 1 || world > 8 || K % 8) return -3;
  for (int i = 0; i < world; ++i)
    if (row_end[i] < (i ? row_end[i - 1] : 0) || row_end[i] > N) return -3;
  if (row_end[world - 1] != N) return -3;
  const int tiles = (N + 255) / 256 + 1;
  cudaError_t e = cudaMemsetAsync(ready, 0, sizeof(int) * tiles,
                                  reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return (int)e;
  g_gather.world = world; g_gather.rank = rank;
  g_gather.ready = (int*)ready;
  for (int i = 0; i < 8; ++i) {
    g_gather.src[i] = i < world ? copies[i] : nullptr;
    g_gather.row_end[i] = i < world ? row_end[i] : N;
  }
  const int r = pf_gemm(A, w_full, C, M, N, K, lda, ldb, ldc, 0, 0, in_dtype, out_dtype, bias,
                        bias_dtype, residual, ldr, aux, ldaux, epilogue, 0, alpha, status,
                        sm_count, 256, stream);
  g_gather = GatherArgs();
  return r;
}

// Convolution as an implicit GEMM (no im2col buffer): y[B*Ho*Wo, Cout] = epi(patches(x) . w2^T)
// with x NHWC [B, H, W, C] and w2 [Cout, KH*KW*C] (taps outermost, channels innermost).  Needs
// C % 64 == 0, 128 % Wo == 0, (Ho * Wo) % 128 == 0 (tiles are whole output rows of one image)
// and stride 1 or 2; returns -3 otherwise so that the caller can take the im2col route.
PF_API int pf_conv_gemm(const void* x, const void* w2, void* y, int B, int H, int W, int C,
                        int Cout, int KH, int KW, int stride, int pad, long long ldw,
                        long long ldy, int in_dtype, int out_dtype, const void* bias,
                        int bias_dtype, const void* residual, long long ldr, int epilogue,
                        int* status, int sm_count, void* stream) {
  const int Ho = (H + 2 * pad - KH) / stride + 1, Wo = (W + 2 * pad - KW) / stride + 1;
  if (C % 64 || Wo <= 0 || Wo > 128 || 128 % Wo || (Ho * Wo) % 128 || (stride != 1 && stride != 2))
    return -3;
  g_conv.on = 1; g_conv.B = B; g_conv.H = H; g_conv.W = W; g_conv.C = C; g_conv.KH = KH;
  g_conv.KW = KW; g_conv.stride = stride; g_conv.pad = pad; g_conv.Ho = Ho; g_conv.Wo = Wo;
  const int r = pf_gemm(x, w2, y, B * Ho * Wo, Cout, KH * KW * C, 0, ldw, ldy, 0, 0, in_dtype,
                        out_dtype, bias, bias_dtype, residual, ldr, nullptr, 0, epilogue, 0, 1.0f,
                        status, sm_count, 0, stream);
  g_conv = ConvArgs();
  return r;
}

// Weight gradient of the same convolution as an implicit GEMM:
// dw2[Cout, KH*KW*C] (+)= dy[B*Ho*Wo, Cout]^T . patches(x), fp32 output; the patches are read
// from x (NHWC) 64 output pixels at a time.  Needs C % 64 == 0, Cout % 8 == 0, Wo dividing 64 or
// a multiple of it, (Ho * Wo) % 64 == 0, stride 1 or 2; returns -3 otherwise.
PF_API int pf_conv_wgrad(const void* dy, const void* x, void* dw2, int B, int H, int W, int C,
                         int Cout, int KH, int KW, int stride, int pad, int in_dtype,
                         int accumulate, int* status, int sm_count, void* stream) {
  const int Ho = (H + 2 * pad - KH) / stride + 1, Wo = (W + 2 * pad - KW) / stride + 1;
  if (C % 64 || Cout % 8 || Wo <= 0 || (64 % Wo && Wo % 64) || (Ho * Wo) % 64 ||
      (stride != 1 && stride != 2))
    return -3;
  g_conv.on = 2; g_conv.B = B; g_conv.H = H; g_conv.W = W; g_conv.C = C; g_conv.KH = KH;
  g_conv.KW = KW; g_conv.stride = stride; g_conv.pad = pad; g_conv.Ho = Ho; g_conv.Wo = Wo;
  const int r = pf_gemm(dy, x, dw2, Cout, KH * KW * C, B * Ho * Wo, Cout, 0,
                        (long long)KH * KW * C, 1, 1, in_dtype, PF_F32, nullptr, 0, nullptr, 0,
                        nullptr, 0, 0, accumulate, 1.0f, status, sm_count, 0, stream);
  g_conv = ConvArgs();
  return r;
}
