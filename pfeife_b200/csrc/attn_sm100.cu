// Flash attention for sm_100a, forward and backward, on tcgen05 tensor cores.
//
// Layout: q [B, Sq, H, D], k/v [B, Sk, H, D] with arbitrary (16-byte aligned) batch / sequence /
// head strides and a unit inner stride, so the three slices of a fused QKV projection are
// consumed in place through 4-D TMA tensor maps.  Head dims up to 128, any multiple of 8
// (88 for ViT-g/14 runs as 96 with zero-filled tails: the tensor map's inner extent is D, so
// the tail of the last 64-element block is filled with zeros by TMA, never with the next head).
//
// Forward: a persistent kernel, one CTA per SM walking over (q tile of 128, head, batch) items,
// with a TMA producer warp (K and V rings), an MMA issuer warp and four softmax warps (thread
// <-> query row <-> TMEM lane); per 128-row K/V tile:
//     S = Q K^T            tcgen05.mma, smem x smem -> one of two S buffers in TMEM; the next
//                          tile's S is issued before this tile's probabilities are waited for
//     online softmax       one tcgen05.ld of S -> registers (base-2 exponent, running max / sum)
//     P -> smem            16-bit, in the 128B-swizzled K-major layout the MMA reads; two buffers
//     O += P V             tcgen05.mma, V in place as an MN-major operand, O accumulated in TMEM
//                          and rescaled there only when the row maximum grew by more than 2^8
// The score matrix never exists in global memory.  (Details at attn_fwd_ws_kernel.)
//
// Backward, one CTA per (k/v tile of 128, head, batch), looping over q tiles, five MMAs per
// tile pair with S/P and dP/dS in TMEM / smem and dK, dV accumulated in TMEM:
//     S = Q K^T ; P = exp2(S*c - lse2) ; dP = dO V^T ; dS = P * (dP - delta) * scale
//     dV += P^T dO ; dK += dS^T Q ; dQ_tile = dS K  -> fp32 atomics into dq_accum
// delta = rowsum(dO * O) comes from a small pre-pass; dq_accum is converted by a post-pass.
//
// Short tails.  A sequence length just above a multiple of 128 (ViT: 257 = 2 x 128 + the class
// token) would spend a whole 128-row query tile on a few rows.  In the forward, when at most
// ATT_TAIL_MAX rows are left over, the tensor-core tiles cover only the full multiples and a
// small CUDA-core kernel computes the leftover query rows.  (The same split of the backward,
// measured on ViT-g/14 shapes, cost more in its leftover-key kernel than the tiles it saved.)
#include <cstdlib>
#include "common.cuh"
#include "api.h"

namespace pf {

constexpr int ATT_BM = 128;   // query rows per tile
constexpr int ATT_BN = 128;   // key rows per tile
constexpr int ATT_BLK = 16384;  // bytes of one [128 rows x 64 x 16-bit] swizzled block
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr int ATT_TAIL_MAX = 4;      // leftover rows handled on CUDA cores
constexpr int ATT_TAIL_SEQ_MAX = 2048;  // longest other dimension the CUDA-core paths stage in smem

struct AttnParams {
  int B, H, Sq, Sk, D;
  int causal;
  float scale;
  int fmt;  // 0 fp16, 1 bf16
  void* o;              // fwd: out [B,Sq,H,D] contiguous
  float* lse;           // [B,H,Sq]
  // backward
  const float* delta;   // [B,H,Sq]
  float* dq_accum;      // [B,Sq,H,D] fp32, zeroed
  void* dk;             // [B,Sk,H,D] with strides sdkv (batch, seq, head)
  void* dv;
  long long sdkv[3];
  int* status;
  // raw views for the CUDA-core tail path of the forward (element strides: batch, seq, head)
  const void* q; const void* k; const void* v;
  long long sq[3], sk[3], sv[3];
  int q_tiles, q_tail;  // tensor-core query tiles; leftover query rows after them
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b),
               "f"(c), "f"(d)
               : "memory");
}

__device__ __forceinline__ float block_reduce(float v, float* red, bool is_max) {
  // red: 32 floats of shared memory; every thread of the CTA calls
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = is_max ? warp_max(v) : warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = is_max ? -INFINITY : 0.f;
  for (int i = 0; i < nw; ++i) r = is_max ? fmaxf(r, red[i]) : r + red[i];
  return r;
}

// dot product of a 16-bit global row (16-byte aligned, D a multiple of 8) with fp32 values in
// shared memory
template <typename T>
__device__ __forceinline__ float dot_row(const T* row, const float* sv, int D) {
  // D <= 128: up to 16 vectors, requested together so that one memory latency covers the row
  uint4 u[16];
  const int nv = D / 8;
#pragma unroll
  for (int c = 0; c < 16; ++c)
    if (c < nv) u[c] = __ldg(reinterpret_cast<const uint4*>(row) + c);
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < 16; ++c) {
    if (c < nv) {
      const T* e = reinterpret_cast<const T*>(&u[c]);
#pragma unroll
      for (int j = 0; j < 8; ++j) s = fmaf(to_f32<T>(e[j]), sv[c * 8 + j], s);
    }
  }
  return s;
}

// acc[0..7] += w * (8 consecutive 16-bit values at `src`)
template <typename T>
__device__ __forceinline__ void axpy8(float (&acc)[8], float w, const uint4& u) {
  const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = fmaf(w, to_f32<T>(e[j]), acc[j]);
}

// Forward for one leftover query row on CUDA cores (128 threads).
template <typename T>
__device__ void attn_fwd_tail_row(const AttnParams& p, uint8_t* smem, int qi, int h, int b) {
  float* qs = reinterpret_cast<float*>(smem);       // [128]
  float* red = qs + 128;                            // [32]
  float* sc = red + 32;                             // [Sk]
  const int tid = threadIdx.x;
  const T* qrow = reinterpret_cast<const T*>(p.q) + b * p.sq[0] + (long long)qi * p.sq[1] +
                  h * p.sq[2];
  for (int d = tid; d < p.D; d += blockDim.x) qs[d] = to_f32<T>(qrow[d]);
  __syncthreads();
  const float c2 = p.scale * LOG2E;
  const int shift = p.Sk - p.Sq;
  const T* kb = reinterpret_cast<const T*>(p.k) + b * p.sk[0] + h * p.sk[2];
  float mx = -INFINITY;
  for (int j = tid; j < p.Sk; j += blockDim.x) {
    const bool vis = !(p.causal && j > qi + shift);
    const float sj = vis ? dot_row<T>(kb + (long long)j * p.sk[1], qs, p.D) * c2 : -INFINITY;
    sc[j] = sj;
    mx = fmaxf(mx, sj);
  }
  mx = block_reduce(mx, red, true);
  const float m_use = (mx == -INFINITY) ? 0.f : mx;
  float sum = 0.f;
  for (int j = tid; j < p.Sk; j += blockDim.x) {
    const float pj = exp2f(sc[j] - m_use);
    sc[j] = pj;
    sum += pj;
  }
  const float l = block_reduce(sum, red, false);    // its barriers also publish sc[]
  const float inv = l > 0.f ? 1.f / l : 0.f;
  {
    // thread = (key group g of 8, column vector cv of 16): keys g, g+8, ... ; 8 columns each
    const int cv = tid & 15, g = tid >> 4;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (cv * 8 < p.D) {
      const T* vb = reinterpret_cast<const T*>(p.v) + b * p.sv[0] + h * p.sv[2] + cv * 8;
      int j = g;
      for (; j + 24 < p.Sk; j += 32) {
        const uint4 u0 = __ldg(reinterpret_cast<const uint4*>(vb + (long long)j * p.sv[1]));
        const uint4 u1 = __ldg(reinterpret_cast<const uint4*>(vb + (long long)(j + 8) * p.sv[1]));
        const uint4 u2 = __ldg(reinterpret_cast<const uint4*>(vb + (long long)(j + 16) * p.sv[1]));
        const uint4 u3 = __ldg(reinterpret_cast<const uint4*>(vb + (long long)(j + 24) * p.sv[1]));
        axpy8<T>(acc, sc[j], u0); axpy8<T>(acc, sc[j + 8], u1);
        axpy8<T>(acc, sc[j + 16], u2); axpy8<T>(acc, sc[j + 24], u3);
      }
      for (; j < p.Sk; j += 8)
        axpy8<T>(acc, sc[j], __ldg(reinterpret_cast<const uint4*>(vb + (long long)j * p.sv[1])));
    }
    __syncthreads();                 // sc[] is dead after this point: reuse it for the fold
    float* fold = sc;                // [8 groups][128 columns]
#pragma unroll
    for (int e = 0; e < 8; ++e) fold[g * 128 + cv * 8 + e] = acc[e];
    __syncthreads();
    if (tid < p.D) {
      float a = 0.f;
#pragma unroll
      for (int gg = 0; gg < 8; ++gg) a += fold[gg * 128 + tid];
      T* dst = reinterpret_cast<T*>(p.o) + (((long long)b * p.Sq + qi) * p.H + h) * p.D;
      dst[tid] = from_f32<T>(a * inv);
    }
  }
  if (tid == 0)
    p.lse[((long long)b * p.H + h) * p.Sq + qi] = (l > 0.f) ? (mx + log2f(l)) * LN2 : -INFINITY;
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Writes 32 consecutive 16-bit values of row `r`, columns [c0, c0+32), into a [128 x 128]
// K-major tile made of two swizzled [128 x 64] blocks.
template <typename T>
__device__ __forceinline__ void store_p_chunk(uint8_t* tile, int r, int c0, const float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = c0 + j * 8;
    const int blk = c >> 6;
    const int chunk = (c & 63) >> 3;
    uint4 q;
    q.x = pack2<T>(v[j * 8 + 0], v[j * 8 + 1]);
    q.y = pack2<T>(v[j * 8 + 2], v[j * 8 + 3]);
    q.z = pack2<T>(v[j * 8 + 4], v[j * 8 + 5]);
    q.w = pack2<T>(v[j * 8 + 6], v[j * 8 + 7]);
    *reinterpret_cast<uint4*>(tile + blk * ATT_BLK + r * 128 + ((chunk ^ (r & 7)) << 4)) = q;
  }
}

// one [128 rows x DP] tile = DP/64 (rounded up) swizzled blocks, loaded with one TMA per block
template <int NBLK>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* map, uint64_t* bar,
                                          int h, int s0, int b) {
  mbar_expect_tx(bar, NBLK * ATT_BLK);
#pragma unroll
  for (int i = 0; i < NBLK; ++i) tma_load_4d(dst + i * ATT_BLK, map, bar, i * 64, h, s0, b);
}

// A[128 x K] (K-major blocks) . B[N x K]^T (K-major blocks), K = KSTEPS * 16
template <int KSTEPS>
__device__ __forceinline__ void mma_kk(uint32_t d_tmem, uint32_t sa, uint32_t sb, uint32_t idesc,
                                       bool accumulate_first) {
#pragma unroll
  for (int k = 0; k < KSTEPS; ++k) {
    const uint32_t off = (k >> 2) * ATT_BLK + (k & 3) * 32;
    tc_mma_f16(d_tmem, make_desc_sw128(sa + off, 16, 1024), make_desc_sw128(sb + off, 16, 1024),
               idesc, (k > 0) || accumulate_first);
  }
}
// A[128 x 128] K-major . B given as [K=128 rows][N] (N contiguous, MN-major blocks of 64)
__device__ __forceinline__ void mma_k_mn(uint32_t d_tmem, uint32_t sa, uint32_t sb, uint32_t idesc,
                                         bool accumulate_first, int ksteps = 8) {
#pragma unroll 1
  for (int k = 0; k < ksteps; ++k) {
    const uint32_t aoff = (k >> 2) * ATT_BLK + (k & 3) * 32;
    tc_mma_f16(d_tmem, make_desc_sw128(sa + aoff, 16, 1024),
               make_desc_sw128(sb + k * 2048, ATT_BLK, 1024), idesc, (k > 0) || accumulate_first);
  }
}
// A given as [K=128 rows][M=128] (M contiguous) . B given as [K=128 rows][N] (N contiguous)
__device__ __forceinline__ void mma_mn_mn(uint32_t d_tmem, uint32_t sa, uint32_t sb, uint32_t idesc,
                                          bool accumulate_first, int ksteps = 8) {
#pragma unroll 1
  for (int k = 0; k < ksteps; ++k) {
    tc_mma_f16(d_tmem, make_desc_sw128(sa + k * 2048, ATT_BLK, 1024),
               make_desc_sw128(sb + k * 2048, ATT_BLK, 1024), idesc, (k > 0) || accumulate_first);
  }
}


// Leftover rows in kernels of their own: small shared memory and block size, so that many of
// these latency-bound CTAs share an SM instead of each holding a tensor-core CTA's resources.
template <typename T>
__global__ void __launch_bounds__(128)
attn_fwd_tail_kernel(const AttnParams p) {
  extern __shared__ uint8_t tail_smem[];
  attn_fwd_tail_row<T>(p, tail_smem, p.q_tiles * ATT_BM + (int)blockIdx.x, blockIdx.y, blockIdx.z);
}
// ================================================================================ forward
// Persistent, warp-specialised forward.  One CTA per SM walks over (q tile, head, batch) work
// items; its 6 warps have fixed roles:
//   warp 0     TMA producer: Q of the item, then K / V tiles into a ring of ST stages; it runs
//              ahead of the consumers, across item boundaries too
//   warp 1     MMA issuer: S_j = Q K_j^T into one of two S buffers in TMEM, O (+)= P_j V_j into
//              the O accumulator in TMEM.  S_{j+1} is issued BEFORE it waits for P_j, so the
//              tensor core computes the next scores while the softmax warps work on this tile
//   warps 2-5  softmax, thread <-> query row <-> TMEM lane: one read of S, running maximum,
//              P = exp2(S c - m) written to shared memory in the layout the P V product reads
// P has two buffers, so a tile's probabilities are computed and stored while the previous
// tile's P V still runs.  O stays in TMEM for the whole item.  The row maximum that scales P is only raised when the
// true maximum has grown by more than 2^8 since it was last set; then the row of O (and the
// running sum) is rescaled in place (tcgen05.ld / st).  P therefore stays below 2^8, which both
// 16-bit formats hold, and most tiles need no rescaling at all.
// TMEM: S0 [0,128) S1 [128,256) O [256, 256+DP) of 512 allocated columns.
template <int DP>
struct FwdCfg {
  static constexpr int NBLK = (DP + 63) / 64;
  static constexpr int TILE = NBLK * ATT_BLK;
  static constexpr int ST = NBLK >= 2 ? 2 : 3;          // K/V ring stages
  static constexpr int OFF_K = TILE;
  static constexpr int OFF_V = OFF_K + ST * TILE;
  static constexpr int OFF_P = OFF_V + ST * TILE;       // two buffers of [128 q][128 kv] 16-bit
  static constexpr int P_BYTES = 2 * ATT_BLK;           // (two swizzled blocks each)
  static constexpr int OFF_BAR = OFF_P + 2 * P_BYTES;
  static constexpr int SMEM = OFF_BAR + 256 + 1024;     // barriers + alignment slack
  static constexpr int THREADS = 192;
};

struct FwdItem {
  int q0, h, b, n_tiles;
};
__device__ __forceinline__ FwdItem fwd_item(const AttnParams& p, int w) {
  FwdItem it;
  // causal: the later query tiles see more keys; they go first so the long items start early
  const int qt = p.causal ? (p.q_tiles - 1 - w % p.q_tiles) : (w % p.q_tiles);
  it.q0 = qt * ATT_BM;
  const int r = w / p.q_tiles;
  it.h = r % p.H;
  it.b = r / p.H;
  int kv_end = p.Sk;
  if (p.causal) kv_end = min(p.Sk, it.q0 + ATT_BM + (p.Sk - p.Sq));
  it.n_tiles = kv_end > 0 ? (kv_end + ATT_BN - 1) / ATT_BN : 0;
  return it;
}

template <typename T, int DP>
__global__ void __launch_bounds__(FwdCfg<DP>::THREADS, 1)
attn_fwd_ws_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                   const __grid_constant__ CUtensorMap tv, const AttnParams p, const int n_items) {
  using C = FwdCfg<DP>;
  constexpr int NBLK = C::NBLK, TILE = C::TILE, ST = C::ST;
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + C::OFF_K;
  uint8_t* sV = smem + C::OFF_V;
  uint8_t* sP = smem + C::OFF_P;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* bar_q_full = bars;            // TMA bytes of Q
  uint64_t* bar_q_empty = bars + 1;       // last S product of the item has read Q
  uint64_t* bar_k_full = bars + 2;        // [ST]
  uint64_t* bar_v_full = bars + 2 + ST;   // [ST]
  uint64_t* bar_k_empty = bars + 2 + 2 * ST;    // [ST] Q K^T of the tile has completed
  uint64_t* bar_v_empty = bars + 2 + 3 * ST;    // [ST] P V of the tile has completed
  uint64_t* bar_s_full = bars + 2 + 4 * ST;     // [2]
  uint64_t* bar_s_empty = bar_s_full + 2;       // [2] the softmax warps hold S in registers
  uint64_t* bar_p_full = bar_s_empty + 2;       // P is in shared memory (and O rescaled)
  uint64_t* bar_pv_done = bar_p_full + 1;       // [2], by tile parity: P V has completed (that P
                                                // buffer is free, O holds every tile up to it)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_pv_done + 2);
  constexpr int N_BARS = 2 + 4 * ST + 7;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    tma_prefetch_desc(&tq); tma_prefetch_desc(&tk); tma_prefetch_desc(&tv);
    for (int i = 0; i < N_BARS; ++i) mbar_init(&bars[i], 1);
    for (int i = 0; i < 2; ++i) mbar_init(&bar_s_empty[i], 4);   // lane 0 of each softmax warp
    mbar_init(bar_p_full, 4);
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_o = tmem + 256;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t g = 0, qc = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
        const FwdItem it = fwd_item(p, w);
        if (it.n_tiles == 0) continue;
        ok = mbar_wait(bar_q_empty, (qc & 1) ^ 1, p.status, PF_ERR_TIMEOUT_EMPTY);
        if (!ok) break;
        load_tile<NBLK>(sQ, &tq, bar_q_full, it.h, it.q0, it.b);
        ++qc;
        // K runs one tile ahead of V: a K stage is free as soon as its Q K^T has completed, a V
        // stage only after its P V, and the next scores are wanted first
        auto load_v = [&](int j, uint32_t gv) -> bool {
          const int st = gv % ST;
          if (!mbar_wait(&bar_v_empty[st], ((gv / ST) & 1) ^ 1, p.status, PF_ERR_TIMEOUT_EMPTY))
            return false;
          load_tile<NBLK>(sV + st * TILE, &tv, &bar_v_full[st], it.h, j * ATT_BN, it.b);
          return true;
        };
        for (int j = 0; j < it.n_tiles && ok; ++j) {
          const uint32_t gk = g + j;
          const int st = gk % ST;
          ok = mbar_wait(&bar_k_empty[st], ((gk / ST) & 1) ^ 1, p.status, PF_ERR_TIMEOUT_EMPTY);
          if (!ok) break;
          load_tile<NBLK>(sK + st * TILE, &tk, &bar_k_full[st], it.h, j * ATT_BN, it.b);
          if (j > 0) ok = load_v(j - 1, gk - 1);
        }
        if (ok) ok = load_v(it.n_tiles - 1, g + it.n_tiles - 1);
        g += it.n_tiles;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_f16(128, 128, p.fmt, 0, 0);
      const uint32_t idesc_o = make_idesc_f16(128, DP, p.fmt, 0, 1);
      uint32_t g = 0, qc = 0;
      bool ok = true;
      // S of global tile `gg` (tile j of the item)
      auto issue_s = [&](uint32_t gg, int j) -> bool {
        const int st = gg % ST, sb = gg & 1;
        if (!mbar_wait(&bar_k_full[st], (gg / ST) & 1, p.status, PF_ERR_TIMEOUT_FULL)) return false;
        if (!mbar_wait(&bar_s_empty[sb], ((gg >> 1) & 1) ^ 1, p.status, PF_ERR_TIMEOUT_TMEM_EMPTY))
          return false;
        tc_fence_after();
        const int rem = min(ATT_BN, p.Sk - j * ATT_BN);
        const int n_mma = (rem + 15) / 16 * 16;
        const uint32_t id = (n_mma == ATT_BN) ? idesc_s : make_idesc_f16(128, n_mma, p.fmt, 0, 0);
        mma_kk<DP / 16>(tmem + sb * 128, smem_u32(sQ), smem_u32(sK + st * TILE), id, false);
        tc_commit(&bar_k_empty[st]);
        tc_commit(&bar_s_full[sb]);
        return true;
      };
      for (int w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
        const FwdItem it = fwd_item(p, w);
        if (it.n_tiles == 0) continue;
        ok = mbar_wait(bar_q_full, qc & 1, p.status, PF_ERR_TIMEOUT_FULL);
        ++qc;
        ok = ok && issue_s(g, 0);
        for (int j = 0; j < it.n_tiles && ok; ++j) {
          const uint32_t gg = g + j;
          if (j + 1 < it.n_tiles) ok = issue_s(gg + 1, j + 1);
          else tc_commit(bar_q_empty);     // every S product of this item has been issued
          if (!ok) break;
          const int st = gg % ST;
          ok = mbar_wait(bar_p_full, gg & 1, p.status, PF_ERR_TIMEOUT_FULL) &&
               mbar_wait(&bar_v_full[st], (gg / ST) & 1, p.status, PF_ERR_TIMEOUT_FULL);
          if (!ok) break;
          tc_fence_after();
          const int rem = min(ATT_BN, p.Sk - j * ATT_BN);
          mma_k_mn(t_o, smem_u32(sP + (gg & 1) * C::P_BYTES), smem_u32(sV + st * TILE), idesc_o,
                   j > 0, (rem + 15) / 16);
          tc_commit(&bar_v_empty[st]);
          tc_commit(&bar_pv_done[gg & 1]);
        }
        g += it.n_tiles;
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax (4 warps)
    const int quad = warp & 3;                       // TMEM lane quadrant of this warp
    const int row = quad * 32 + lane;
    const uint32_t lane_off = uint32_t(quad * 32) << 16;
    const float c2 = p.scale * LOG2E;
    const int shift = p.Sk - p.Sq;
    uint32_t g = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
      const FwdItem it = fwd_item(p, w);
      const int qi = it.q0 + row;
      T* dst = reinterpret_cast<T*>(p.o) + (((long long)it.b * p.Sq + qi) * p.H + it.h) * p.D;
      float* lse_dst = p.lse + ((long long)it.b * p.H + it.h) * p.Sq + qi;
      if (it.n_tiles == 0) {       // no key is visible to this query tile
        if (qi < p.Sq) {
          for (int c = 0; c < p.D / 8; ++c) reinterpret_cast<uint4*>(dst)[c] = make_uint4(0, 0, 0, 0);
          *lse_dst = -INFINITY;
        }
        continue;
      }
      float m_used = -INFINITY, l = 0.f;
      for (int j = 0; j < it.n_tiles && ok; ++j) {
        const uint32_t gg = g + j;
        const int sb = gg & 1;
        const int k0 = j * ATT_BN;
        const int rem = min(ATT_BN, p.Sk - k0);
        const int n_chunks = ((rem + 15) / 16 * 16 + 31) / 32;
        // a tile needs masks when it is ragged or crosses the causal diagonal of this q tile
        const bool masked = rem < ATT_BN || (p.causal && k0 + ATT_BN - 1 > it.q0 + shift);
        ok = mbar_wait(&bar_s_full[sb], (gg >> 1) & 1, p.status, PF_ERR_TIMEOUT_TMEM_FULL);
        if (!ok) break;
        tc_fence_after();
        uint32_t s[4][32];
        const uint32_t t_s = tmem + sb * 128 + lane_off;
#pragma unroll
        for (int c = 0; c < 4; ++c)
          if (c < n_chunks) tmem_ld32(t_s + c * 32, s[c]);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_s_empty[sb]);
        float mx = -INFINITY;
        if (!masked) {
          // full tile: four independent chains, no visibility tests
          float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              m0 = fmaxf(m0, __uint_as_float(s[c][i]));
              m1 = fmaxf(m1, __uint_as_float(s[c][i + 1]));
              m2 = fmaxf(m2, __uint_as_float(s[c][i + 2]));
              m3 = fmaxf(m3, __uint_as_float(s[c][i + 3]));
            }
          }
          mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (c < n_chunks) {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const int kj = k0 + c * 32 + i;
                const bool vis = kj < p.Sk && !(p.causal && kj > qi + shift);
                if (vis) mx = fmaxf(mx, __uint_as_float(s[c][i]));
              }
            }
          }
        }
        mx *= c2;                                   // c2 > 0; -inf stays -inf
        float alpha = 1.f;
        if (j == 0) {
          m_used = mx;
        } else if (mx > m_used + 8.f) {             // also true when m_used is still -inf
          alpha = exp2f(m_used - mx);               // exp2(-inf) = 0: nothing had accumulated
          m_used = mx;
        }
        const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;
        // This tile's P buffer was last read by the P V of the tile before the previous one
        // (any item): long done, so the probabilities below are computed while the previous
        // tile's P V still runs.  (Parity of the phase before this tile's own on that barrier;
        // on a fresh barrier the wait passes.)
        uint8_t* sPj = sP + (gg & 1) * C::P_BYTES;
        ok = mbar_wait(&bar_pv_done[gg & 1], ((gg >> 1) & 1) ^ 1, p.status,
                       PF_ERR_TIMEOUT_TMEM_FULL);
        if (!ok) break;
        if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
          // rare: the row maximum grew by more than 2^8.  O must hold every earlier tile of
          // the item before it is rescaled: wait for the previous tile's P V
          ok = mbar_wait(&bar_pv_done[(gg - 1) & 1], ((gg - 1) >> 1) & 1, p.status,
                         PF_ERR_TIMEOUT_TMEM_FULL);
          if (!ok) break;
          tc_fence_after();
          {
#pragma unroll
            for (int c = 0; c < DP / 32; ++c) {
              uint32_t o[32];
              tmem_ld32(t_o + lane_off + c * 32, o);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st32(t_o + lane_off + c * 32, o);
            }
            tmem_st_wait();
          }
        }
        float rs = 0.f;
        if (!masked) {
          float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;
          const float nm = -m_sub;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            float pv[32];
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              pv[i] = exp2f(fmaf(__uint_as_float(s[c][i]), c2, nm));
              pv[i + 1] = exp2f(fmaf(__uint_as_float(s[c][i + 1]), c2, nm));
              pv[i + 2] = exp2f(fmaf(__uint_as_float(s[c][i + 2]), c2, nm));
              pv[i + 3] = exp2f(fmaf(__uint_as_float(s[c][i + 3]), c2, nm));
              r0 += pv[i]; r1 += pv[i + 1]; r2 += pv[i + 2]; r3 += pv[i + 3];
            }
            store_p_chunk<T>(sPj, row, c * 32, pv);
          }
          rs = (r0 + r1) + (r2 + r3);
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (c < n_chunks) {
              float pv[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const int kj = k0 + c * 32 + i;
                const bool vis = kj < p.Sk && !(p.causal && kj > qi + shift);
                pv[i] = vis ? exp2f(fmaf(__uint_as_float(s[c][i]), c2, -m_sub)) : 0.f;
                rs += pv[i];
              }
              store_p_chunk<T>(sPj, row, c * 32, pv);
            }
          }
        }
        l = l * alpha + rs;
        fence_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_p_full);
      }
      if (!ok) break;
      g += it.n_tiles;
      // ---- epilogue of the item: O / l
      ok = mbar_wait(&bar_pv_done[(g - 1) & 1], ((g - 1) >> 1) & 1, p.status,
                     PF_ERR_TIMEOUT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
      for (int c = 0; c < DP / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(t_o + lane_off + c * 32, o);
        tmem_ld_wait();
        if (qi < p.Sq) {
#pragma unroll
          for (int v8 = 0; v8 < 4; ++v8) {
            if (c * 32 + v8 * 8 < p.D) {
              uint4 q;
              q.x = pack2<T>(__uint_as_float(o[v8 * 8 + 0]) * inv, __uint_as_float(o[v8 * 8 + 1]) * inv);
              q.y = pack2<T>(__uint_as_float(o[v8 * 8 + 2]) * inv, __uint_as_float(o[v8 * 8 + 3]) * inv);
              q.z = pack2<T>(__uint_as_float(o[v8 * 8 + 4]) * inv, __uint_as_float(o[v8 * 8 + 5]) * inv);
              q.w = pack2<T>(__uint_as_float(o[v8 * 8 + 6]) * inv, __uint_as_float(o[v8 * 8 + 7]) * inv);
              reinterpret_cast<uint4*>(dst)[c * 4 + v8] = q;
            }
          }
        }
      }
      if (qi < p.Sq) *lse_dst = (l > 0.f) ? (m_used + log2f(l)) * LN2 : -INFINITY;
      // the reads of O above have completed (tcgen05.wait::ld); the next item's first P V,
      // which overwrites O, is ordered after them by this warp's next arrival on bar_p_full
      tc_fence_before();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

// ================================================================================ backward
// delta[b,h,i] = sum_d dO[b,i,h,d] * O[b,i,h,d]
template <typename T>
__global__ void __launch_bounds__(128)
attn_delta_kernel(const T* __restrict__ dout, const T* __restrict__ out, float* __restrict__ delta,
                  int B, int S, int H, int D) {
  // eight lanes per row, 16-byte loads (D is a multiple of 8): four rows per warp
  const int lane = threadIdx.x & 31, sub = lane & 7;
  const long long row = ((long long)blockIdx.x * 4 + (threadIdx.x >> 5)) * 4 + (lane >> 3);
  const bool live = row < (long long)B * S * H;
  float s = 0.f;
  if (live) {
    const uint4* a = reinterpret_cast<const uint4*>(dout + row * D);
    const uint4* c = reinterpret_cast<const uint4*>(out + row * D);
    for (int i = sub; i < D / 8; i += 8) {
      const uint4 ua = __ldg(a + i), uc = __ldg(c + i);
      const T* ea = reinterpret_cast<const T*>(&ua);
      const T* ec = reinterpret_cast<const T*>(&uc);
#pragma unroll
      for (int j = 0; j < 8; ++j) s = fmaf(to_f32<T>(ea[j]), to_f32<T>(ec[j]), s);
    }
  }
  s += __shfl_xor_sync(0xffffffffu, s, 4);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  if (live && sub == 0) {
    const int h = (int)(row % H);
    const long long bs = row / H;
    const int i = (int)(bs % S);
    const long long b = bs / S;
    delta[(b * H + h) * S + i] = s;
  }
}

// dq[b, i, h, :] (strided) = convert(acc[b, i, h, :]) ; acc is contiguous [B*Sq*H, D]
template <typename T>
__global__ void __launch_bounds__(256)
attn_dq_convert_kernel(const float* __restrict__ acc, T* __restrict__ dq, long long rows, int D,
                       int Sq, int H, long long sb, long long ss, long long sh) {
  const int dv = D / 8;
  const long long total = rows * dv;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long row = i / dv;
    const int c = (int)(i - row * dv);
    const int h = (int)(row % H);
    const long long bs = row / H;
    const int si = (int)(bs % Sq);
    const long long b = bs / Sq;
    const float4 a0 = reinterpret_cast<const float4*>(acc + row * D)[2 * c];
    const float4 a1 = reinterpret_cast<const float4*>(acc + row * D)[2 * c + 1];
    uint4 q;
    q.x = pack2<T>(a0.x, a0.y); q.y = pack2<T>(a0.z, a0.w);
    q.z = pack2<T>(a1.x, a1.y); q.w = pack2<T>(a1.z, a1.w);
    reinterpret_cast<uint4*>(dq + b * sb + (long long)si * ss + (long long)h * sh)[c] = q;
  }
}

template <typename T, int DP>
__global__ void __launch_bounds__(256)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                const AttnParams p) {
  constexpr int NBLK = (DP + 63) / 64;
  constexpr int TILE = NBLK * ATT_BLK;
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  // Q / dO tiles: two stages when a tile is one block (head dim <= 64), so that the next query
  // tile travels while this one is worked on; larger head dims leave room for one stage only
  constexpr int QST = (NBLK == 1) ? 2 : 1;
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE;
  uint8_t* sQ0 = sV + TILE;                  // [QST] tiles
  uint8_t* sdO0 = sQ0 + QST * TILE;          // [QST] tiles
  uint8_t* sP = sdO0 + QST * TILE;           // [q][kv] 16-bit, 2 blocks
  uint8_t* sdS = sP + 2 * ATT_BLK;           // [q][kv] 16-bit, 2 blocks
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + 2 * ATT_BLK);
  uint64_t* bar_kv = bars, *bar_q = bars + 1 /* [2] */, *bar_mma1 = bars + 3, *bar_mma2 = bars + 4,
          *bar_dq = bars + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row_t = (warp & 3) * 32 + lane;     // TMEM lane / tile row of this thread
  const int half = warp >> 2;                   // which half of the columns this warp handles
  const int k0 = blockIdx.x * ATT_BN, h = blockIdx.y, b = blockIdx.z;
  if (tid == 0) {
    tma_prefetch_desc(&tq); tma_prefetch_desc(&tk); tma_prefetch_desc(&tv);
    tma_prefetch_desc(&tdo);
    for (int i = 0; i < 6; ++i) mbar_init(&bars[i], 1);
    mbar_fence_init();
  }
  if (warp == 0) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_s = tmem, t_dp = tmem + 128, t_dv = tmem + 256, t_dk = tmem + 384;
  const uint32_t lane_off = uint32_t((warp & 3) * 32) << 16;

  const uint32_t idesc_s = make_idesc_f16(128, 128, p.fmt, 0, 0);     // Q K^T and dO V^T
  const uint32_t idesc_kd = make_idesc_f16(128, DP, p.fmt, 1, 1);     // P^T dO, dS^T Q
  const uint32_t idesc_dq = make_idesc_f16(128, DP, p.fmt, 0, 1);     // dS K
  const float c2 = p.scale * LOG2E;
  const int shift = p.Sk - p.Sq;

  const int rem_k = min(ATT_BN, p.Sk - k0);
  const int nk_mma = (rem_k + 15) / 16 * 16;          // key columns that exist, rounded to 16
  const int nk_chunks = (nk_mma + 31) / 32;
  const uint32_t idesc_sr = make_idesc_f16(128, nk_mma, p.fmt, 0, 0);
  int q_begin = 0;
  if (p.causal) q_begin = max(0, k0 - shift) / ATT_BM * ATT_BM;   // first q tile that sees k0
  const int n_q = (p.Sq + ATT_BM - 1) / ATT_BM;

  if (tid == 0) {
    mbar_expect_tx(bar_kv, 2 * TILE);
#pragma unroll
    for (int i = 0; i < NBLK; ++i) {
      tma_load_4d(sK + i * ATT_BLK, &tk, bar_kv, i * 64, h, k0, b);
      tma_load_4d(sV + i * ATT_BLK, &tv, bar_kv, i * 64, h, k0, b);
    }
  }
  bool ok = true;
  uint32_t ph = 0;
  bool first = true;
  int it = 0;                                  // iteration count: stage and phase of Q / dO
  auto load_q = [&](int stage, int q_row) {
    mbar_expect_tx(&bar_q[stage], 2 * TILE);
#pragma unroll
    for (int i = 0; i < NBLK; ++i) {
      tma_load_4d(sQ0 + stage * TILE + i * ATT_BLK, &tq, &bar_q[stage], i * 64, h, q_row, b);
      tma_load_4d(sdO0 + stage * TILE + i * ATT_BLK, &tdo, &bar_q[stage], i * 64, h, q_row, b);
    }
  };
  for (int qt = q_begin / ATT_BM; qt < n_q && ok; ++qt, ++it) {
    const int q0 = qt * ATT_BM;
    const int qi = q0 + row_t;
    const int qs = (QST == 2) ? (it & 1) : 0;
    uint8_t* sQ = sQ0 + qs * TILE;
    uint8_t* sdO = sdO0 + qs * TILE;
    if (tid == 0) {
      if (first) load_q(qs, q0);   // later tiles are requested ahead (below)
      // two stages: the other stage was last read by the products of the previous iteration,
      // which have completed (this thread waited for them), so the next tile is requested now
      if (QST == 2 && qt + 1 < n_q) load_q(qs ^ 1, q0 + ATT_BM);
      if (first) ok = mbar_wait(bar_kv, 0, p.status, PF_ERR_TIMEOUT_FULL);
      ok = ok && mbar_wait(&bar_q[qs], (QST == 2) ? ((it >> 1) & 1) : ph, p.status,
                           PF_ERR_TIMEOUT_FULL);
      if (ok) {
        tc_fence_after();
        mma_kk<DP / 16>(t_s, smem_u32(sQ), smem_u32(sK), idesc_sr, false);    // S  = Q K^T
        mma_kk<DP / 16>(t_dp, smem_u32(sdO), smem_u32(sV), idesc_sr, false);  // dP = dO V^T
        tc_commit(bar_mma1);
      }
    }
    __syncwarp();
    // the row statistics travel from global memory while the first two products run
    const bool row_ok = qi < p.Sq;
    const float lse2 = row_ok ? __ldg(p.lse + ((long long)b * p.H + h) * p.Sq + qi) * LOG2E : 0.f;
    const float dl = row_ok ? __ldg(p.delta + ((long long)b * p.H + h) * p.Sq + qi) : 0.f;
    ok = mbar_wait(bar_mma1, ph, p.status, PF_ERR_TIMEOUT_TMEM_FULL);
    if (!ok) break;
    tc_fence_after();
    // rows of P / dS that the products below read: the query rows that exist, rounded up to 16;
    // a warp whose 32 rows all lie beyond them has nothing to write
    const int q_rows = (min(ATT_BM, p.Sq - q0) + 15) / 16 * 16;
    const bool warp_has_rows = (warp & 3) * 32 < q_rows;
    const bool tile_masked = rem_k < ATT_BN || q0 + ATT_BM > p.Sq ||
                             (p.causal && k0 + ATT_BN - 1 > q0 + shift);
#pragma unroll 1
    for (int c = half; c < nk_chunks && warp_has_rows; c += 2) {
      uint32_t rs[32], rp[32];
      tmem_ld32(t_s + lane_off + c * 32, rs);
      tmem_ld32(t_dp + lane_off + c * 32, rp);
      tmem_ld_wait();
      float pv[32], ds[32];
      if (!tile_masked) {       // full tile away from the causal diagonal: no visibility tests
        const float nl = -lse2;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float pr = exp2f(fmaf(__uint_as_float(rs[i]), c2, nl));
          pv[i] = pr;
          ds[i] = pr * (__uint_as_float(rp[i]) - dl) * p.scale;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int kj = k0 + c * 32 + i;
          const bool vis = row_ok && kj < p.Sk && !(p.causal && kj > qi + shift);
          const float pr = vis ? exp2f(__uint_as_float(rs[i]) * c2 - lse2) : 0.f;
          pv[i] = pr;
          ds[i] = pr * (__uint_as_float(rp[i]) - dl) * p.scale;
        }
      }
      store_p_chunk<T>(sP, row_t, c * 32, pv);
      store_p_chunk<T>(sdS, row_t, c * 32, ds);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      // sP / sdS hold [q rows][kv cols]: as A operands of the two products below they are
      // MN-major (M = kv contiguous within a row, K = q across rows)
      // reductions run only over the query rows / key columns that exist (rounded to 16);
      // rows of dV / dK beyond the last key are never stored
      const int q_steps = (min(ATT_BM, p.Sq - q0) + 15) / 16;
      mma_mn_mn(t_dv, smem_u32(sP), smem_u32(sdO), idesc_kd, !first, q_steps);  // dV += P^T dO
      mma_mn_mn(t_dk, smem_u32(sdS), smem_u32(sQ), idesc_kd, !first, q_steps);  // dK += dS^T Q
      tc_commit(bar_mma2);
      mma_k_mn(t_s, smem_u32(sdS), smem_u32(sK), idesc_dq, false, nk_mma / 16);  // dQ = dS K
      tc_commit(bar_dq);
    }
    __syncwarp();
    ok = mbar_wait(bar_dq, ph, p.status, PF_ERR_TIMEOUT_TMEM_FULL);
    if (!ok) break;
    tc_fence_after();
    if (QST == 1 && tid == 0 && qt + 1 < n_q) {
      // every MMA that read sQ / sdO has completed (commits complete in issue order): the next
      // tile's loads overlap the dQ reduction below
      load_q(0, q0 + ATT_BM);
    }
    {
      // the TMEM loads are warp-collective: every lane executes them, only valid rows add
      float* dst = p.dq_accum + (((long long)b * p.Sq + (row_ok ? qi : 0)) * p.H + h) * p.D;
#pragma unroll
      for (int c = 0; c < DP / 32; ++c) {
        if ((c & 1) != half) continue;            // warp-uniform
        uint32_t raw[32];
        tmem_ld32(t_s + lane_off + c * 32, raw);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            if (c * 32 + i < p.D)                 // D is a multiple of 8
              red_add_v4(dst + c * 32 + i, __uint_as_float(raw[i]), __uint_as_float(raw[i + 1]),
                         __uint_as_float(raw[i + 2]), __uint_as_float(raw[i + 3]));
        }
      }
    }
    ok = mbar_wait(bar_mma2, ph, p.status, PF_ERR_TIMEOUT_TMEM_FULL);
    if (!ok) break;
    ph ^= 1;
    first = false;
    tc_fence_before();
    __syncthreads();
  }

  // epilogue: dK, dV rows of this tile
  if (ok && !first) {
    tc_fence_after();
    const int kj = k0 + row_t;
    const long long off_kv = (long long)b * p.sdkv[0] + (long long)kj * p.sdkv[1] +
                             (long long)h * p.sdkv[2];
    T* dkp = reinterpret_cast<T*>(p.dk) + off_kv;
    T* dvp = reinterpret_cast<T*>(p.dv) + off_kv;
#pragma unroll
    for (int c = 0; c < DP / 32; ++c) {
      if ((c & 1) != half) continue;              // warp-uniform
      uint32_t rk[32], rv[32];
      tmem_ld32(t_dk + lane_off + c * 32, rk);
      tmem_ld32(t_dv + lane_off + c * 32, rv);
      tmem_ld_wait();
      if (kj < p.Sk) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int d0 = c * 32 + g * 8;
          if (d0 < p.D) {
            uint4 a, bq;
            a.x = pack2<T>(__uint_as_float(rk[g * 8 + 0]), __uint_as_float(rk[g * 8 + 1]));
            a.y = pack2<T>(__uint_as_float(rk[g * 8 + 2]), __uint_as_float(rk[g * 8 + 3]));
            a.z = pack2<T>(__uint_as_float(rk[g * 8 + 4]), __uint_as_float(rk[g * 8 + 5]));
            a.w = pack2<T>(__uint_as_float(rk[g * 8 + 6]), __uint_as_float(rk[g * 8 + 7]));
            bq.x = pack2<T>(__uint_as_float(rv[g * 8 + 0]), __uint_as_float(rv[g * 8 + 1]));
            bq.y = pack2<T>(__uint_as_float(rv[g * 8 + 2]), __uint_as_float(rv[g * 8 + 3]));
            bq.z = pack2<T>(__uint_as_float(rv[g * 8 + 4]), __uint_as_float(rv[g * 8 + 5]));
            bq.w = pack2<T>(__uint_as_float(rv[g * 8 + 6]), __uint_as_float(rv[g * 8 + 7]));
            *reinterpret_cast<uint4*>(dkp + d0) = a;
            *reinterpret_cast<uint4*>(dvp + d0) = bq;
          }
        }
      }
    }
  } else if (ok && first) {
    // no query tile sees this key tile (causal with Sk > Sq + ...): gradients are zero
    const int kj = k0 + row_t;
    if (kj < p.Sk && half == 0) {
      const long long off_kv = (long long)b * p.sdkv[0] + (long long)kj * p.sdkv[1] +
                               (long long)h * p.sdkv[2];
      T* dkp = reinterpret_cast<T*>(p.dk) + off_kv;
      T* dvp = reinterpret_cast<T*>(p.dv) + off_kv;
      for (int d = 0; d < p.D; ++d) { dkp[d] = from_f32<T>(0.f); dvp[d] = from_f32<T>(0.f); }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

// ------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn attn_get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) ==
            cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// [B, S, H, D] view with element strides (sb, ss, sh, 1); box = 64 x 1 x 128 x 1
static int make_tmap_bshd(CUtensorMap* map, const void* base, int fmt, int B, int S, int H, int D,
                          long long sb, long long ss, long long sh) {
  EncodeTiledFn enc = attn_get_encode();
  if (!enc) return -100;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)sh * 2, (cuuint64_t)ss * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {64, 1, 128, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, fmt ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                   4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(1000 + (int)r);
}

// `done` must be a distinct array per kernel instantiation (kernels of equal signature share
// one function-pointer type), so the callers own it.
template <typename K>
static int set_smem(K kern, int bytes, bool* done) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 0 && dev < 64) done[dev] = true;
  }
  return 0;
}

static int attn_sm_count() {
  static int sms[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (!sms[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    sms[dev] = n;
  }
  return sms[dev];
}

template <typename T, int DP>
static int launch_fwd_ws(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                         const AttnParams& p, cudaStream_t st) {
  using C = FwdCfg<DP>;
  auto kern = attn_fwd_ws_kernel<T, DP>;
  static bool done[64] = {};
  int r = set_smem(kern, C::SMEM, done);
  if (r) return r;
  const int n_items = p.q_tiles * p.H * p.B;
  if (n_items > 0) {
    const int sms = attn_sm_count();
    kern<<<n_items < sms ? n_items : sms, C::THREADS, C::SMEM, st>>>(tq, tk, tv, p, n_items);
    PF_CHECK_LAUNCH();
  }
  if (p.q_tail > 0) {
    // [q 128 | red 32 | scores max(Sk, 8 x 128 for the fold)] floats
    const int bytes = (160 + (p.Sk > 1024 ? p.Sk : 1024)) * 4;
    attn_fwd_tail_kernel<T><<<dim3(p.q_tail, p.H, p.B), 128, bytes, st>>>(p);
    PF_CHECK_LAUNCH();
  }
  return 0;
}

template <typename T, int DP>
static int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                      const CUtensorMap& tdo, const AttnParams& p, cudaStream_t st) {
  constexpr int NBLK = (DP + 63) / 64;
  constexpr int SMEM = (NBLK == 1 ? 6 : 4) * NBLK * ATT_BLK + 4 * ATT_BLK + 128 + 1024;
  auto kern = attn_bwd_kernel<T, DP>;
  static bool done[64] = {};
  int r = set_smem(kern, SMEM, done);
  if (r) return r;
  dim3 grid((p.Sk + ATT_BN - 1) / ATT_BN, p.H, p.B);
  kern<<<grid, 256, SMEM, st>>>(tq, tk, tv, tdo, p);
  PF_CHECK_LAUNCH();
  return 0;
}

static bool strides_ok(const void* ptr, long long sb, long long ss, long long sh) {
  return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && sb % 8 == 0 && ss % 8 == 0 && sh % 8 == 0;
}

// Tensor-core tiles and leftover rows of a sequence of length S: a short leftover (at most
// ATT_TAIL_MAX rows after at least one full tile) goes to the CUDA-core paths, which stage the
// other sequence dimension (`other`) in shared memory; otherwise the last tile is ragged.
static void split_tail(int S, int other, int* tiles, int* tail) {
  const int left = S % ATT_BM;
  if (S > ATT_BM && left > 0 && left <= ATT_TAIL_MAX && other <= ATT_TAIL_SEQ_MAX) {
    *tiles = S / ATT_BM;
    *tail = left;
  } else {
    *tiles = (S + ATT_BM - 1) / ATT_BM;
    *tail = 0;
  }
}

static void set_views(AttnParams& p, const void* q, const void* k, const void* v,
                      const long long* sq, const long long* sk, const long long* sv) {
  p.q = q; p.k = k; p.v = v;
  for (int i = 0; i < 3; ++i) { p.sq[i] = sq[i]; p.sk[i] = sk[i]; p.sv[i] = sv[i]; }
}

}  // namespace pf

using namespace pf;

#define PF_ATTN_DISPATCH(FN, ...)                                              \
  do {                                                                         \
    const int DP = (D + 31) / 32 * 32;                                         \
    if (dtype == PF_F16) {                                                     \
      switch (DP) {                                                            \
        case 32: return FN<__half, 32>(__VA_ARGS__);                            \
        case 64: return FN<__half, 64>(__VA_ARGS__);                            \
        case 96: return FN<__half, 96>(__VA_ARGS__);                            \
        case 128: return FN<__half, 128>(__VA_ARGS__);                          \
      }                                                                        \
    } else {                                                                   \
      switch (DP) {                                                            \
        case 32: return FN<__nv_bfloat16, 32>(__VA_ARGS__);                     \
        case 64: return FN<__nv_bfloat16, 64>(__VA_ARGS__);                     \
        case 96: return FN<__nv_bfloat16, 96>(__VA_ARGS__);                     \
        case 128: return FN<__nv_bfloat16, 128>(__VA_ARGS__);                   \
      }                                                                        \
    }                                                                          \
    return -3;                                                                 \
  } while (0)

// strides are in elements, order (batch, seq, head) for each of q, k, v
PF_API int pf_attn_fwd(const void* q, const void* k, const void* v, void* o, void* lse, int B,
                       int H, int Sq, int Sk, int D, const long long* sq, const long long* sk,
                       const long long* sv, int causal, float scale, int dtype, int* status,
                       void* stream) {
  if (dtype != PF_F16 && dtype != PF_BF16) return -1;
  if (D % 8 || D > 128) return -3;
  if (!strides_ok(q, sq[0], sq[1], sq[2]) || !strides_ok(k, sk[0], sk[1], sk[2]) ||
      !strides_ok(v, sv[0], sv[1], sv[2]))
    return -2;
  const int fmt = dtype == PF_BF16;
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = make_tmap_bshd(&tq, q, fmt, B, Sq, H, D, sq[0], sq[1], sq[2]))) return r;
  if ((r = make_tmap_bshd(&tk, k, fmt, B, Sk, H, D, sk[0], sk[1], sk[2]))) return r;
  if ((r = make_tmap_bshd(&tv, v, fmt, B, Sk, H, D, sv[0], sv[1], sv[2]))) return r;
  AttnParams p = {};
  p.B = B; p.H = H; p.Sq = Sq; p.Sk = Sk; p.D = D; p.causal = causal; p.scale = scale;
  p.fmt = fmt; p.o = o; p.lse = (float*)lse; p.status = status;
  set_views(p, q, k, v, sq, sk, sv);
  split_tail(Sq, Sk, &p.q_tiles, &p.q_tail);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  PF_ATTN_DISPATCH(launch_fwd_ws, tq, tk, tv, p, st);
}

// dout / out: [B, Sq, H, D] contiguous; dq_accum fp32 [B,Sq,H,D] (zeroed here); dq, dk, dv
// contiguous outputs; delta fp32 [B,H,Sq] scratch.
PF_API int pf_attn_bwd(const void* dout, const void* q, const void* k, const void* v,
                       const void* out, const void* lse, void* delta, void* dq_accum, void* dq,
                       void* dk, void* dv, int B, int H, int Sq, int Sk, int D,
                       const long long* sq, const long long* sk, const long long* sv,
                       const long long* sdq, const long long* sdkv, int causal,
                       float scale, int dtype, int* status, int sm_count, void* stream) {
  if (dtype != PF_F16 && dtype != PF_BF16) return -1;
  if (D % 8 || D > 128) return -3;
  if (!strides_ok(q, sq[0], sq[1], sq[2]) || !strides_ok(k, sk[0], sk[1], sk[2]) ||
      !strides_ok(v, sv[0], sv[1], sv[2]) || (reinterpret_cast<uintptr_t>(dout) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15) ||
      !strides_ok(dq, sdq[0], sdq[1], sdq[2]) || !strides_ok(dk, sdkv[0], sdkv[1], sdkv[2]) ||
      !strides_ok(dv, sdkv[0], sdkv[1], sdkv[2]))
    return -2;
  const int fmt = dtype == PF_BF16;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long rows = (long long)B * Sq * H;
  if (dtype == PF_F16)
    attn_delta_kernel<__half><<<(unsigned)((rows + 15) / 16), 128, 0, st>>>(
        (const __half*)dout, (const __half*)out, (float*)delta, B, Sq, H, D);
  else
    attn_delta_kernel<__nv_bfloat16><<<(unsigned)((rows + 15) / 16), 128, 0, st>>>(
        (const __nv_bfloat16*)dout, (const __nv_bfloat16*)out, (float*)delta, B, Sq, H, D);
  PF_CHECK_LAUNCH();
  cudaMemsetAsync(dq_accum, 0, sizeof(float) * rows * D, st);
  CUtensorMap tq, tk, tv, tdo;
  int r;
  if ((r = make_tmap_bshd(&tq, q, fmt, B, Sq, H, D, sq[0], sq[1], sq[2]))) return r;
  if ((r = make_tmap_bshd(&tk, k, fmt, B, Sk, H, D, sk[0], sk[1], sk[2]))) return r;
  if ((r = make_tmap_bshd(&tv, v, fmt, B, Sk, H, D, sv[0], sv[1], sv[2]))) return r;
  if ((r = make_tmap_bshd(&tdo, dout, fmt, B, Sq, H, D, (long long)Sq * H * D, (long long)H * D,
                          D)))
    return r;
  AttnParams p = {};
  p.B = B; p.H = H; p.Sq = Sq; p.Sk = Sk; p.D = D; p.causal = causal; p.scale = scale;
  p.fmt = fmt; p.lse = (float*)const_cast<void*>(lse); p.delta = (const float*)delta;
  p.dq_accum = (float*)dq_accum; p.dk = dk; p.dv = dv; p.status = status;
  p.sdkv[0] = sdkv[0]; p.sdkv[1] = sdkv[1]; p.sdkv[2] = sdkv[2];
  {
    auto run = [&]() -> int { PF_ATTN_DISPATCH(launch_bwd, tq, tk, tv, tdo, p, st); };
    if ((r = run())) return r;
  }
  const long long n = rows * (D / 8);
  long long blocks = (n + 255) / 256;
  const long long cap = (long long)(sm_count > 0 ? sm_count : 148) * 8;
  if (blocks > cap) blocks = cap;
  if (dtype == PF_F16)
    attn_dq_convert_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(
        (const float*)dq_accum, (__half*)dq, rows, D, Sq, H, sdq[0], sdq[1], sdq[2]);
  else
    attn_dq_convert_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(
        (const float*)dq_accum, (__nv_bfloat16*)dq, rows, D, Sq, H, sdq[0], sdq[1], sdq[2]);
  PF_CHECK_LAUNCH();
  return 0;
}
