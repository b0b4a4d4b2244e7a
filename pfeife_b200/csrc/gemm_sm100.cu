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
// TMEM lane quadrant and split the tile's columns, which halves the epilogue latency per tile).
#include <cstring>
#include "common.cuh"
#include "api.h"

namespace pf {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;       // 64 x 16-bit = one 128 B swizzle row
constexpr int GEMM_UMMA_K = 16;
constexpr int GEMM_EPI_WARPS = 8;     // two warps per TMEM lane quadrant, half the columns each
constexpr int GEMM_GATHER_WARPS = 2;  // copy remote rows of a sharded B operand (fused all-gather)
constexpr int GEMM_THREADS = 64 + 32 * (GEMM_EPI_WARPS + GEMM_GATHER_WARPS);

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
  // ---- fused all-gather of the B operand (weights sharded by rows over `gather_world` ranks)
  int gather_world;            // 0: B is an ordinary local operand
  int gather_rank;
  int gather_rows;             // rows of B owned by each rank
  const void* gather_src[8];   // peer pointers to every rank's shard [gather_rows, K] (pitch ldb)
  void* gather_dst;            // local full-size B [N, K] (pitch ldb); own rows already in place
  int* gather_ready;           // local counters, one per BN-row tile of B, zeroed before launch
  long long gather_ld;
};

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  // epilogue staging for TMA stores: per epilogue warp one [32 rows x 32 cols] box for C and one
  // for aux (16-bit outputs) or one 4 KB box for C (fp32 outputs)
  static constexpr int STAGING_OFFSET = BAR_OFFSET + 1024;
  static constexpr int STAGING_PER_WARP = 4096;
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

template <typename OutT, int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                    const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_c,
                    const __grid_constant__ CUtensorMap tmap_aux, const GemmParams p) {
  using S = GemmSmem<BN, STAGES>;
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
  constexpr uint32_t TMEM_COLS = 2 * BN;  // 256 or 512: a power of two

  const int num_m = (p.M + GEMM_BM - 1) / GEMM_BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + GEMM_BK - 1) / GEMM_BK;
  // with a fused all-gather the tiles whose rows of B this rank owns are computed first, while
  // the remote rows are still arriving
  const int n_rot = p.gather_world > 1 ? (p.gather_rank * p.gather_rows) / BN : 0;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 32 * GEMM_EPI_WARPS);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % num_m) * GEMM_BM;
        const int nt = (tile / num_m + n_rot) % num_n;
        const int n0 = nt * BN;
        if (p.gather_world > 1) {
          // rows of this B tile that other ranks own must have landed in the local buffer
          int expect = 0;
          for (int r = n0; r < min(p.N, n0 + BN); ++r)
            expect += (r / p.gather_rows) != p.gather_rank;
          long long t0 = clock64();
          while (*reinterpret_cast<volatile int*>(p.gather_ready + nt) < expect) {
            if (clock64() - t0 > PF_WAIT_CYCLES) { report(p.status, PF_ERR_TIMEOUT_PEER_FLAG); ok = false; break; }
          }
          __threadfence();
          asm volatile("fence.proxy.async;" ::: "memory");   // generic writes -> TMA reads
          if (!ok) break;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, p.status, PF_ERR_TIMEOUT_EMPTY);
          if (!ok) break;
          uint8_t* sa = smem + stage * S::STAGE_BYTES;
          uint8_t* sb = sa + S::A_BYTES;
          mbar_expect_tx(&full_bar[stage], S::STAGE_BYTES);
          const int k0 = kb * GEMM_BK;
          if (!p.a_mn) {
            tma_load_2d(sa, &tmap_a, &full_bar[stage], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < GEMM_BM / 64; ++j)
              tma_load_2d(sa + j * 8192, &tmap_a, &full_bar[stage], m0 + j * 64, k0);
          }
          if (!p.b_mn) {
            tma_load_2d(sb, &tmap_b, &full_bar[stage], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * 8192, &tmap_b, &full_bar[stage], n0 + j * 64, k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(GEMM_BM, BN, p.fmt, p.a_mn, p.b_mn);
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
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        ok = mbar_wait(&tmem_empty[acc], acc_phase ^ 1, p.status, PF_ERR_TIMEOUT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, p.status, PF_ERR_TIMEOUT_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < GEMM_BK / GEMM_UMMA_K; ++k) {
            const uint64_t da = make_desc_sw128(sa + k * a_adv, a_lbo, 1024);
            const uint64_t db = make_desc_sw128(sb + k * b_adv, b_lbo, 1024);
            tc_mma_f16(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          tc_commit(&empty_bar[stage]);  // smem slot reusable once these MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(&tmem_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
    __syncwarp();
  } else if (warp >= 2 + GEMM_EPI_WARPS) {
    // ------------------------------------------------------------------ gather warps
    if (p.gather_world > 1) {
      // All-gather of the remote shards of B: the gather warps of every CTA copy whole
      // rows from the owners' memory (plain peer loads, 16 bytes per lane) into the local
      // buffer and bumps the counter of the row's tile.  The TMA producer of a tile waits for
      // its counter, so the transfer overlaps the tiles computed before it.
      const int ew = blockIdx.x * GEMM_GATHER_WARPS + (warp - 2 - GEMM_EPI_WARPS);
      const int n_ew = gridDim.x * GEMM_GATHER_WARPS;
      const int kvec = p.K / 8;
      for (int r = ew; r < p.N; r += n_ew) {
        const int owner = r / p.gather_rows;
        if (owner == p.gather_rank) continue;
        const uint4* src = reinterpret_cast<const uint4*>(
            reinterpret_cast<const uint16_t*>(p.gather_src[owner]) +
            (long long)(r - owner * p.gather_rows) * p.gather_ld);
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
        if (lane == 0) atomicAdd(p.gather_ready + r / BN, 1);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (8 warps)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const int col_half = (warp - 2) >> 2;          // which half of the tile's columns
    const int c_begin = col_half * (BN / 2), c_end = c_begin + BN / 2;
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    OutT* C = reinterpret_cast<OutT*>(p.C);
    const OutT* R = reinterpret_cast<const OutT*>(p.residual);
    OutT* AUX = reinterpret_cast<OutT*>(p.aux);
    uint8_t* stage_c = smem + S::STAGING_OFFSET + (warp - 2) * S::STAGING_PER_WARP;
    uint8_t* stage_aux = stage_c + 2048;           // only used by 16-bit outputs
    const bool aux_out = AUX && (p.epilogue == EPI_GELU || p.epilogue == EPI_GELU_TANH ||
                                 p.epilogue == EPI_SILU);
    bool stores_pending = false;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int m0 = (tile % num_m) * GEMM_BM;
      const int n0 = ((tile / num_m + n_rot) % num_n) * BN;
      ok = mbar_wait(&tmem_full[acc], acc_phase, p.status, PF_ERR_TIMEOUT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + row_in_tile;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + (uint32_t(quad * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = c_begin; c < c_end; c += 32) {
        const int col = n0 + c;
        if (col >= p.N) break;  // uniform across the warp
        uint32_t raw[32];
        tmem_ld32(t_row + c, raw);
        tmem_ld_wait();
        const int nvalid = min(32, p.N - col);
        const bool vec = p.vec_ok != 0;
        const bool tma_out = p.tma_store != 0;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]) * p.alpha;
        if (p.bias) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i < nvalid) v[i] += load_bias(p.bias, p.bias_dtype, col + i);
        }
        if (tma_out && stores_pending) {
          // the previous chunk's TMA stores must have read the staging boxes before reuse
          if (lane == 0) tma_store_wait_read();
          __syncwarp();
          stores_pending = false;
        }
        if (p.epilogue == EPI_GELU || p.epilogue == EPI_GELU_TANH || p.epilogue == EPI_SILU) {
          if (aux_out) {
            if (tma_out) stage_row32<OutT>(stage_aux, lane, v);
            else if (row_ok)
              store_row32<OutT>(AUX + (long long)row * p.ldaux + col, vec, nvalid, v);
          }
          if (p.epilogue == EPI_GELU) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = gelu_erf(v[i]);
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
            for (int i = 0; i < 32; ++i) v[i] *= dgelu_erf(z[i]);
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
            tma_store_commit();
          }
          stores_pending = true;
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
      mbar_arrive(&tmem_empty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  // teardown: every role reaches this point (all waits are bounded)
  if (warp >= 2 && lane == 0 && p.tma_store) tma_store_wait_all();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
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

template <typename OutT, int BN, int STAGES>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                       const CUtensorMap& taux, const GemmParams& p, int sm_count,
                       cudaStream_t stream) {
  using S = GemmSmem<BN, STAGES>;
  auto kern = gemm_tcgen05_kernel<OutT, BN, STAGES>;
  static bool configured[64] = {};  // the attribute is per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const int num_tiles = ((p.M + GEMM_BM - 1) / GEMM_BM) * ((p.N + BN - 1) / BN);
  const int grid = num_tiles < sm_count ? num_tiles : sm_count;
  kern<<<grid, GEMM_THREADS, S::TOTAL, stream>>>(ta, tb, tc, taux, p);
  PF_CHECK_LAUNCH();
  return 0;
}

}  // namespace pf

using namespace pf;

// all-gather arguments of the call in flight on this thread (set by pf_gemm_allgather)
struct GatherArgs { int world = 0, rank = 0, rows = 0; int* ready = nullptr; const void* src[8] = {}; };
static thread_local GatherArgs g_gather;

PF_API int pf_gemm(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                   long long ldb, long long ldc, int a_mn, int b_mn, int in_dtype, int out_dtype,
                   const void* bias, int bias_dtype, const void* residual, long long ldr,
                   void* aux, long long ldaux, int epilogue, int accumulate, float alpha,
                   int* status, int sm_count, int tile_n, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (in_dtype != PF_F16 && in_dtype != PF_BF16) return -1;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15))
    return -2;  // TMA needs 16-byte aligned bases and pitches
  const int fmt = in_dtype == PF_BF16 ? 1 : 0;
  const int tn = tile_n & 1023;     // bit 10 of tile_n forces the direct-store epilogue (tests)
  const int BN = (tn == 128 || tn == 256) ? tn : (N <= 128 ? 128 : 256);

  CUtensorMap ta, tb;
  int r;
  if (!a_mn) r = make_tmap_2d_16bit(&ta, A, fmt, K, M, lda, GEMM_BK, GEMM_BM);
  else       r = make_tmap_2d_16bit(&ta, A, fmt, M, K, lda, 64, GEMM_BK);
  if (r) return r;
  if (!b_mn) r = make_tmap_2d_16bit(&tb, B, fmt, K, N, ldb, GEMM_BK, BN);
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
  p.gather_rows = g_gather.rows; p.gather_dst = const_cast<void*>(B);
  p.gather_ready = g_gather.ready; p.gather_ld = ldb;
  for (int i = 0; i < 8; ++i) p.gather_src[i] = g_gather.src[i];
  const size_t es = out_dtype == PF_F32 ? 4 : 2;
  auto aligned = [&](const void* ptr, long long ld) {
    return ptr == nullptr || ((reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && (ld * es) % 16 == 0);
  };
  p.vec_ok = aligned(C, ldc) && aligned(residual, ldr) && aligned(aux, ldaux);
  // TMA-store epilogue: needs aligned outputs; fp32 accumulation uses the reduce-add store,
  // 16-bit accumulation (unused by the framework) stays on the direct path
  p.tma_store = p.vec_ok && !(accumulate && out_dtype != PF_F32) && !(tile_n & 1024) &&
                !(aux && out_dtype == PF_F32);
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
  if (sm_count <= 0) sm_count = 148;

#define PF_GEMM_DISPATCH(T)                                                          \
  (BN == 256 ? launch_gemm<T, 256, 4>(ta, tb, tc, taux, p, sm_count, st)             \
             : launch_gemm<T, 128, 6>(ta, tb, tc, taux, p, sm_count, st))
  switch (out_dtype) {
    case PF_F32: return PF_GEMM_DISPATCH(float);
    case PF_F16: return PF_GEMM_DISPATCH(__half);
    case PF_BF16: return PF_GEMM_DISPATCH(__nv_bfloat16);
  }
  return -1;
}

// Diagnostic: result of encoding a 2-D 16-bit tensor map with the given geometry (0 = ok).
PF_API int pf_tmap_probe(const void* base, long long inner, long long outer, long long ld,
                         int box_inner, int box_outer) {
  CUtensorMap m;
  return make_tmap_2d_16bit(&m, base, 1, inner, outer, ld, box_inner, box_outer);
}

// C[M,N] = epi(A[M,K] . W[N,K]^T) where W is sharded by rows over `world` ranks: rank r owns rows
// [r*rows_per_rank, (r+1)*rows_per_rank) and `shards[r]` is a pointer (peer-mapped for r != rank)
// to its [rows_per_rank, K] shard with pitch ldb.  `w_full` is a local [N, K] buffer (pitch ldb)
// that already holds this rank's rows; the kernel fills in the others while it computes.
// `ready` is an int array with one entry per 256-row tile of W (zeroed here).
PF_API int pf_gemm_allgather(const void* A, void* w_full, void* const* shards, int world, int rank,
                             int rows_per_rank, void* ready, void* C, int M, int N, int K,
                             long long lda, long long ldb, long long ldc, int in_dtype,
                             int out_dtype, const void* bias, int bias_dtype,
                             const void* residual, long long ldr, void* aux, long long ldaux,
                             int epilogue, float alpha, int* status, int sm_count, void* stream) {
  if (world < 1 || world > 8 || K % 8) return -3;
  const int tiles = (N + 255) / 256;
  cudaError_t e = cudaMemsetAsync(ready, 0, sizeof(int) * tiles,
                                  reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return (int)e;
  g_gather.world = world; g_gather.rank = rank; g_gather.rows = rows_per_rank;
  g_gather.ready = (int*)ready;
  for (int i = 0; i < 8; ++i) g_gather.src[i] = i < world ? shards[i] : nullptr;
  const int r = pf_gemm(A, w_full, C, M, N, K, lda, ldb, ldc, 0, 0, in_dtype, out_dtype, bias,
                        bias_dtype, residual, ldr, aux, ldaux, epilogue, 0, alpha, status,
                        sm_count, 256, stream);
  g_gather = GatherArgs();
  return r;
}
