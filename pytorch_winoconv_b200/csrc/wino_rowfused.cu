// Row-piece DWM forward for f16 / bf16 on sm_100a (stride 1; the caller presents stride 2 as a stride-1 problem over
// phase channels, see RowDesc): the kernel is decomposed the DWM way into
// 1 x 3 pieces -- along W every run of three taps is a Winograd F(2,3) window (zero taps where the kernel
// ends), along H (and depth) every tap is its own piece, for which F(m,1) is the identity.  All pieces write
// the same four Winograd positions of a tile of 1 x 2 outputs, so they are summed where the GEMM accumulates:
//
//     M[j][tile][k] = sum_{kd,kh,w} sum_c  V_w[row(tile) + kh][colpair(tile)][j][c] * U[kd][kh][w][j][k][c]
//     y[tile][0] = M0 + M1 + M2,   y[tile][1] = M1 - M2 - M3
//
// Why this shape on B200: with both MMA operands in shared memory a narrow accumulator (2-D F(2x2,3x3) needs 16
// positions, i.e. N = 32 columns each in the 512-column TMEM) is bound by the A-operand read, not by the tensor
// pipe.  Four positions leave N = 128, and the tap along H costs nothing to form: a 128-tile block is 8 (or 16)
// output rows x 16 (or 8) column pairs, the transformed slab holds all input rows of the block once, and tap kh
// is the same slab read through a descriptor that starts kh row-groups later.
//
// One persistent CTA per SM; per work item (tile block x 64/128 output channels):
//   warp 0       TMA: raw input patch (5-D box, zero fill = padding) per 32-channel slab
//   warps 1-10   F(2,3) along W on the patch: raw -> four [rows x 32] slabs, 64-byte swizzle, fence.proxy.async
//   warp 11      TMA: transformed-filter slabs of the current (kd, kh, window), four positions per stage
//   warps 12-15  tcgen05.mma (M = 128, N = BN, K = 16) issue + commits, one position each; warp 12: TMEM alloc
//   warps 16-23  epilogue (lane quarter x column half): tcgen05.ld, A^T along W, bias / ReLU / 2x2 max-pool (row partner by shuffle), 32-byte stores
// V and M never exist in global memory.  Every mbarrier wait is bounded and reports through the error word.
// With a batch of two or more and streamed filter slabs the CTAs run as pairs (clusters of two, cta_group::2):
// one M = 256 MMA covers the tile blocks of both, and each loads only its half of every filter slab.
//
// Reference counterparts: the whole chain of src/base_conv_launchers.cu:338-381 (inputNorm2WinoTransform,
// cublas batched GEMM, outputWino2NormTransform, outputAggregate) and the piece table of
// src/base_conv_launchers.h:58-388, here with 1 x 3 pieces.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <map>
#include <mutex>
#include <utility>

#include "wino_common.cuh"
#include "wino_launch.h"

namespace wino {

__device__ unsigned int g_row_error = 0;

namespace rowf {

constexpr int BM = 128;            // tiles per block == TMEM lanes
constexpr int KC = 32;             // reduction slab (channels): 64-byte rows
constexpr int UMMA_K = 16;
constexpr int N_PROD = 320;        // 10 producer warps: a slab set of 160 rows x 4 vectors is two full rounds
constexpr int B_WARP = 1 + N_PROD / 32;   // filter loader
constexpr int MMA_WARP0 = B_WARP + 1;    // first of the MMA-issuing warps
constexpr int N_THREADS = 768;     // 24 warps
constexpr int EPI_WARP0 = 16;      // first of the eight epilogue warps (a multiple of 4: warp & 3 = TMEM lane quarter)
constexpr int N_MMA_THREADS = 4;   // MMA issuers: one per Winograd position (its own accumulator columns)
constexpr long long WAIT_LIMIT_CLOCKS = 2000000000LL;

enum ErrCode : unsigned {
  ERR_RAW_EMPTY = 0x301, ERR_PROD_RAW = 0x302, ERR_PROD_A = 0x303, ERR_B_EMPTY = 0x304, ERR_MMA_ACC = 0x305,
  ERR_MMA_A = 0x306, ERR_MMA_B = 0x307, ERR_EPI = 0x308
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile unsigned *abort_word, unsigned code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  unsigned polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    // the abort word and the clock are looked at every 32nd failed poll: twenty waiting warps that read shared
    // memory on every poll take load/store slots from the producers
    if ((++polls & 31u) != 0u) continue;
    if (*abort_word != 0u) return false;
    if (clock64() - start > WAIT_LIMIT_CLOCKS) {
      *abort_word = code;
      atomicCAS(&g_row_error, 0u, code);
      return false;
    }
  }
  return true;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}
// Shared-memory operand descriptors (reduction-major, 64-byte rows, SWIZZLE_64B: eight-row groups 512 B apart) are
// given as (low word, high word): the high word is a constant of the layout, so an issuing thread only does 32-bit
// adds on the low words between MMAs.
constexpr uint32_t DESC_HI_SW64 = (uint32_t)(512 >> 4) | (1u << 14) | (4u << 29);
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr) { return ((saddr & 0x3FFFFu) >> 4) | (1u << 16); }
__device__ __forceinline__ void umma_f16_lohi(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
      ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(DESC_HI_SW64), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Warp-uniform wait: every lane polls, the outcome is voted.  The single-thread roles (TMA issue, MMA issue) run their
// loops with the whole warp converged and predicate only the issuing instructions on lane 0: a lone lane looping
// while its 31 siblings sit at the final barrier pays ~200 clocks at every taken branch.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile unsigned *abort_word, unsigned code) {
  const bool ok = mbar_wait(bar, parity, abort_word, code);
  return __all_sync(0xffffffffu, ok);
}

// ---- CTA pairs (cluster of two, tcgen05 cta_group::2): one MMA spans both SMs (M = 256: 128 tiles from each), each
// SM loads only its half of every filter slab, so the filter bytes an SM pulls from L2 per multiply-add halve.
// The even CTA of the pair (rank 0) issues the MMAs; barriers it waits on collect arrivals from both CTAs.
// Shared-memory addresses of a cluster carry the CTA rank in bit 24: clearing it names the same offset in rank 0.
constexpr uint32_t PEER_BIT_MASK = 0xFEFFFFFFu;
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_rank0(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar & PEER_BIT_MASK) : "memory");
}
// filter slab load of a pair: both CTAs issue it for their own half; the bytes are counted on rank 0's barrier
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar & PEER_BIT_MASK), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void umma_f16_lohi_pair(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n\t}"
      ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(DESC_HI_SW64), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier at this offset in both CTAs once the MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(mask) : "memory");
}
__device__ __forceinline__ void tmem_ld_x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
}

// two fp32 values in one 64-bit register, and the packed adds of sm_100 on them
__device__ __forceinline__ uint64_t pack_f32x2(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t sub_f32x2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

template <typename T> struct P2;
template <> struct P2<__half> {
  using V = __half2;
  static __device__ __forceinline__ V from(float a, float b) { return __floats2half2_rn(a, b); }
  // (lo, hi) fp32 pair -> packed 16-bit pair, lo in the low half
  static __device__ __forceinline__ uint32_t round_pair(uint64_t v) {
    uint32_t r;
    asm("{\n\t.reg .f32 lo, hi;\n\tmov.b64 {lo, hi}, %1;\n\tcvt.rn.f16x2.f32 %0, hi, lo;\n\t}" : "=r"(r) : "l"(v));
    return r;
  }
  static __device__ __forceinline__ uint32_t max2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("max.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
  }
};
template <> struct P2<__nv_bfloat16> {
  using V = __nv_bfloat162;
  static __device__ __forceinline__ V from(float a, float b) { return __floats2bfloat162_rn(a, b); }
  static __device__ __forceinline__ uint32_t round_pair(uint64_t v) {
    uint32_t r;
    asm("{\n\t.reg .f32 lo, hi;\n\tmov.b64 {lo, hi}, %1;\n\tcvt.rn.bf16x2.f32 %0, hi, lo;\n\t}" : "=r"(r) : "l"(v));
    return r;
  }
  static __device__ __forceinline__ uint32_t max2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("max.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
  }
};
template <typename T> struct __align__(16) V8 { typename P2<T>::V h[4]; };
template <typename T> __device__ __forceinline__ V8<T> v8_add(const V8<T> &a, const V8<T> &b) {
  V8<T> r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.h[i] = __hadd2(a.h[i], b.h[i]);
  return r;
}
template <typename T> __device__ __forceinline__ V8<T> v8_sub(const V8<T> &a, const V8<T> &b) {
  V8<T> r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.h[i] = __hsub2(a.h[i], b.h[i]);
  return r;
}

// 16 consecutive output channels of one pixel, already packed to 16-bit pairs.  mode 2: one 32-byte store (K a
// multiple of 16, 32-byte aligned output) -- a warp's store touches one line per lane whatever its width, so wider
// stores halve the time the epilogue spends in the load/store unit; mode 1: 16-byte stores; mode 0: element-wise.
template <typename T>
__device__ __forceinline__ void store16p(T *dst, const uint32_t (&pk)[8], int kbase, int K, int mode) {
  if (mode == 2) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]),
                 "r"(pk[3]), "r"(pk[4]), "r"(pk[5]), "r"(pk[6]), "r"(pk[7]) : "memory");
  } else if (mode == 1) {
    *reinterpret_cast<uint4 *>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    if (kbase + 8 < K) *reinterpret_cast<uint4 *>(dst + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
  } else {
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      if (kbase + c < K) {
        const unsigned short bits = (unsigned short)((pk[c >> 1] >> ((c & 1) * 16)) & 0xFFFFu);
        *reinterpret_cast<unsigned short *>(dst + c) = bits;
      }
    }
  }
}

// Shared-memory carve-up computed on the host and passed in (all offsets from the 1024-aligned base).
struct Smem {
  int raw_bytes, a_bytes, b_stage_bytes;   // one raw patch; one set of four slabs; one stage of four filter slabs
  int n_b_stages, n_a_bufs;
  int b_group;                             // filter stages per full / empty barrier pair (1, or all kH rows of a window)
  int off_raw[2], off_a[3], off_b, off_bars;
  int total;
};


struct RGeom {
  int N, C, K;
  int Cp;                 // channels of the (padded) input the TMA map addresses
  int D, H, W, oD, oH, oW, yH, yW;
  int pD, pH, pW, kD, kH, kW;
  int PW;                 // F(2,3) windows along W: ceil(kW / 3)
  int RB, CBW;            // tile block: RB output rows x CBW column pairs, RB * CBW == 128
  int MB;                 // tile blocks per work item, stacked along H (they share every filter slab)
  int n_rb, n_cb;         // blocks per image plane
  int slab_rows;          // (MB * RB + kH - 1) * CBW
  int patch_h, patch_w;   // raw patch extents (pixels)
  int n_chunks;           // ceil(C / 32)
  int n_nblocks;
  long long n_items;
  unsigned epilogue;
  // Few-channel input read as it lies (C < 8, e.g. RGB): the TMA map addresses x as [N, D, H, W * C], a patch row
  // is raw_row_el consecutive elements starting at a multiple of eight, the first patch pixel raw_off elements in.
  // A stride-2 layer over few channels is read the same way: the phase channels of one pixel of the stride-1 problem
  // are raw_seg = fW * C0 consecutive elements in each of raw_fh = fH consecutive rows of x.
  // A stride-2 layer whose channel count is a multiple of 32 is read from the caller's tensor through a map that
  // traverses H and W with an element stride of 2: one load fetches one polyphase part of a patch, i.e. exactly the
  // 32-channel step (phase, channel chunk) of the stride-1 problem over phase channels.
  int s2_chunks;          // 0: off; else 32-channel chunks per polyphase part (C0 / 32)
  int s2_fh, s2_fw, s2_pd, s2_ph, s2_pw;   // phases per dimension and the caller's padding
  int raw_c;              // 0: the map addresses [N, D, H, W, Cp]; else the channels of the stride-1 problem (raw_fh * raw_seg)
  int raw_off, raw_row_el;
  int raw_seg, raw_fh;    // elements per pixel and row of x (C, or fW * C0); rows of x per patch row (1, or fH)
  int raw_pd, raw_ph, raw_pw;   // padding of x in its own coordinates (rows, and elements along W), the caller's for a strided layer
};

template <typename T, int BN, int MB, bool PAIR>
__global__ void __launch_bounds__(N_THREADS, 1) rowfused_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                 const __grid_constant__ CUtensorMap map_u,
                                                                 T *__restrict__ y, const T *__restrict__ bias,
                                                                 const __grid_constant__ RGeom g,
                                                                 const __grid_constant__ Smem sl, uint32_t idesc) {
  constexpr int ACC_COLS = MB * 4 * BN;                  // MB blocks x 4 positions x BN columns per buffer
  constexpr int ACC_BUFS = (ACC_COLS <= 256) ? 2 : 1;
  extern __shared__ uint8_t smem_raw_[];
  const uint32_t raw0 = smem_u32(smem_raw_);
  const uint32_t base = (raw0 + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw_ + (base - raw0);
  // barriers: raw_full[2] raw_empty[2] (4 unused) b_full[8] b_empty[8] acc_full[2] acc_empty[2] a_full[3] a_empty[3]
  const uint32_t bars = base + sl.off_bars;
  auto raw_full = [&](int i) { return bars + 8u * i; };
  auto raw_empty = [&](int i) { return bars + 8u * (2 + i); };
  auto a_full = [&](int i) { return bars + 8u * (28 + i); };
  auto a_empty = [&](int i) { return bars + 8u * (31 + i); };
  auto b_full = [&](int i) { return bars + 8u * (8 + i); };
  auto b_empty = [&](int i) { return bars + 8u * (16 + i); };
  auto acc_full = [&](int i) { return bars + 8u * (24 + i); };
  auto acc_empty = [&](int i) { return bars + 8u * (26 + i); };
  volatile unsigned *abort_word = reinterpret_cast<volatile unsigned *>(base_ptr + sl.off_bars + 512);
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(base_ptr + sl.off_bars + 516);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(raw_full(i), 1);
      mbar_init(raw_empty(i), N_PROD / 32);                      // one arrival per producer warp
      mbar_init(acc_full(i), N_MMA_THREADS);                     // one commit per MMA-issuing thread
      mbar_init(acc_empty(i), PAIR ? 16 : 8);                    // one arrival per epilogue warp
    }
    for (int i = 0; i < 3; ++i) {
      mbar_init(a_full(i), PAIR ? 2 * (N_PROD / 32) : N_PROD / 32);
      mbar_init(a_empty(i), N_MMA_THREADS);
    }
    for (int i = 0; i < 8; ++i) {
      mbar_init(b_full(i), 1);
      mbar_init(b_empty(i), N_MMA_THREADS);
    }
    *abort_word = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  if (PAIR) {   // barriers of both CTAs exist before either allocates or arrives remotely
    __syncthreads();
    cluster_sync_all();
  }
  if (warp == MMA_WARP0) {
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void *)tmem_slot)), "r"(512u) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void *)tmem_slot)), "r"(512u) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (PAIR) cluster_sync_all();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  // work items of this CTA (of this pair): the two CTAs of a pair take images 2n and 2n + 1 of the same item
  const long long item0 = PAIR ? (long long)(blockIdx.x >> 1) : (long long)blockIdx.x;
  const long long item_step = PAIR ? (long long)(gridDim.x >> 1) : (long long)gridDim.x;

  // item -> (n, od, rb, cb, nb); the channel block is the fastest index so consecutive CTAs share a patch.  The roles
  // that need the coordinates walk them as mixed-radix digits (first item and the stride are split once with
  // divisions; every further item is five add-with-carry steps, not eight 64-bit divisions).
  struct ItemWalk {
    int nb, cb, rb, od, n5;          // digits of the current item (n5: image, or image pair)
    int s_nb, s_cb, s_rb, s_od, s_n; // digits of the stride
    int r_nb, r_cb, r_rb, r_od;      // radices
    __device__ __forceinline__ void split(long long v, int &a, int &b, int &c, int &d, int &e) const {
      a = (int)(v % r_nb); v /= r_nb;
      b = (int)(v % r_cb); v /= r_cb;
      c = (int)(v % r_rb); v /= r_rb;
      d = (int)(v % r_od); v /= r_od;
      e = (int)v;
    }
    __device__ __forceinline__ void init(long long first, long long step, int n_nb, int n_cb, int n_rb, int n_od) {
      r_nb = n_nb; r_cb = n_cb; r_rb = n_rb; r_od = n_od;
      split(first, nb, cb, rb, od, n5);
      split(step, s_nb, s_cb, s_rb, s_od, s_n);
    }
    __device__ __forceinline__ void advance() {
      int c;
      nb += s_nb;     c = nb >= r_nb; nb -= c ? r_nb : 0;
      cb += s_cb + c; c = cb >= r_cb; cb -= c ? r_cb : 0;
      rb += s_rb + c; c = rb >= r_rb; rb -= c ? r_rb : 0;
      od += s_od + c; c = od >= r_od; od -= c ? r_od : 0;
      n5 += s_n + c;
    }
  };
  auto make_walk = [&]() {
    ItemWalk wk;
    wk.init(item0, item_step, g.n_nblocks, g.n_cb, g.n_rb, g.oD);
    return wk;
  };
  const int steps_per_item = g.kD * g.n_chunks;          // raw patches per item
  // When one channel block covers K and a whole item's filter slabs fit the stage ring, they are loaded once and
  // stay: stage index = slab position within the item, no refills.
  const bool b_resident = g.n_nblocks == 1 && steps_per_item * g.PW * g.kH <= sl.n_b_stages;

  if (warp == 0) {
    // ---------------------------------------------------------------- raw input patches
    {
      uint32_t it = 0;
      bool alive = true;
      ItemWalk wk = make_walk();
      for (long long item = item0; item < g.n_items && alive; item += item_step, wk.advance()) {
        const int n = PAIR ? 2 * wk.n5 + (int)rank : wk.n5, od = wk.od, rb = wk.rb, cb = wk.cb;
        for (int kd = 0; kd < g.kD && alive; ++kd)
          for (int ch = 0; ch < g.n_chunks; ++ch) {
            const int s = it & 1;
            if (!mbar_wait_warp(raw_empty(s), ((it >> 1) & 1u) ^ 1u, abort_word, ERR_RAW_EMPTY)) { alive = false; break; }
            if (lane == 0) {
              mbar_expect_tx(raw_full(s), (uint32_t)sl.raw_bytes);
              if (g.raw_c)   // rows of W * C elements: start at the multiple of eight at or below the first patch pixel
                tma_load_4d(base + sl.off_raw[s], &map_x, raw_full(s), cb * g.CBW * 2 * g.raw_seg - g.raw_pw - g.raw_off,
                            rb * (MB * g.RB) * g.raw_fh - g.raw_ph, od + kd - g.raw_pd, n);
              else if (g.s2_chunks) {   // step ch = (polyphase part, channel chunk): origin of that part in the caller's tensor
                const int phase = ch / g.s2_chunks, cch = ch - phase * g.s2_chunks;
                const int ph_h = phase / g.s2_fw, ph_w = phase - ph_h * g.s2_fw;
                tma_load_5d(base + sl.off_raw[s], &map_x, raw_full(s), cch * KC, g.s2_fw * (cb * g.CBW * 2) + ph_w - g.s2_pw,
                            g.s2_fh * (rb * (MB * g.RB)) + ph_h - g.s2_ph, od + kd - g.s2_pd, n);
              } else
                tma_load_5d(base + sl.off_raw[s], &map_x, raw_full(s), ch * KC, cb * g.CBW * 2 - g.pW, rb * (MB * g.RB) - g.pH,
                            od + kd - g.pD, n);
            }
            ++it;
          }
      }
      // After an abort nobody consumes the patches still in flight: let them land (bounded) before the CTA can exit.
      if (*abort_word != 0u && lane == 0)
        for (uint32_t back = 1; back <= 2u && back <= it; ++back) {
          const uint32_t j = it - back;
          for (int polls = 0; polls < (1 << 16) && !mbar_try_wait(raw_full((int)(j & 1u)), (j >> 1) & 1u); ++polls) { }
        }
    }
  } else if (warp < B_WARP) {
    // ---------------------------------------------------------------- F(2,3) along W: raw patch -> four slabs
    const int ptid = threadIdx.x - 32;                 // 0..N_PROD-1
    const int n_tasks = g.slab_rows;                   // one task = one slab row (input row, column pair) x one vector
    uint32_t it_raw = 0, it_a = 0;
    int as = 0;
    uint32_t a_par = 1u;                               // parity of the "slab set is free" wait: first round passes
    const int cbw_shift = g.CBW == 16 ? 4 : 3;         // CBW is 16 or 8
    bool alive = true;
    for (long long item = item0; item < g.n_items && alive; item += item_step) {
      for (int step = 0; step < steps_per_item && alive; ++step) {
        const int rs = it_raw & 1;
        // lane 0 polls, the warp follows: the outcome is uniform, so the warp stays converged for the elected arrivals
        unsigned ok = 0;
        if (lane == 0) ok = mbar_wait(raw_full(rs), (it_raw >> 1) & 1u, abort_word, ERR_PROD_RAW) ? 1u : 0u;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (ok == 0u) { alive = false; break; }
        const uint8_t *raw = base_ptr + sl.off_raw[rs];
        // A slab with at most 16 real channels (few-channel input, phase-gathered RGB, the tail of C) is read by the
        // MMAs through one K = 16 step, i.e. the first two 16-byte vectors of each row: only those are produced, and
        // a vector past the last real channel is written as zeros without touching the patch.
        const int ch0 = (step % g.n_chunks) * KC;
        const bool narrow = g.Cp - ch0 <= UMMA_K;
        const int vshift = narrow ? 1 : 2;
        const int v = ptid & ((1 << vshift) - 1);           // 16-byte vector of the 32-channel slab
        const bool real = ch0 + v * 8 < g.Cp;
        for (int w = 0; w < g.PW && alive; ++w) {
          ok = 0;
          if (lane == 0) ok = mbar_wait(a_empty(as), a_par, abort_word, ERR_PROD_A) ? 1u : 0u;
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (ok == 0u) { alive = false; break; }
          uint8_t *slab = base_ptr + sl.off_a[as];
          const int slab_bytes = g.slab_rows * 64;
          const int task_stride = N_PROD >> vshift;
          int row_first = ptid >> vshift;
          if (real && !g.raw_c) {
            // the usual case, two slab rows per round: the eight loads of both rows are in flight together (how fast a
            // slab set is refilled after the MMAs release it bounds the kernel when only two sets fit shared memory)
            for (; row_first + task_stride < n_tasks; row_first += 2 * task_stride) {
              const int row_a = row_first, row_b = row_first + task_stride;
              const int ir_a = row_a >> cbw_shift, cp_a = row_a - (ir_a << cbw_shift);
              const int ir_b = row_b >> cbw_shift, cp_b = row_b - (ir_b << cbw_shift);
              const uint8_t *src_a = raw + ((size_t)(ir_a * g.patch_w + 2 * cp_a + 3 * w) * KC + v * 8) * 2;
              const uint8_t *src_b = raw + ((size_t)(ir_b * g.patch_w + 2 * cp_b + 3 * w) * KC + v * 8) * 2;
              V8<T> a0, a1, a2, a3, b0, b1, b2, b3;
              *reinterpret_cast<uint4 *>(&a0) = *reinterpret_cast<const uint4 *>(src_a);
              *reinterpret_cast<uint4 *>(&a1) = *reinterpret_cast<const uint4 *>(src_a + KC * 2);
              *reinterpret_cast<uint4 *>(&a2) = *reinterpret_cast<const uint4 *>(src_a + 2 * KC * 2);
              *reinterpret_cast<uint4 *>(&a3) = *reinterpret_cast<const uint4 *>(src_a + 3 * KC * 2);
              *reinterpret_cast<uint4 *>(&b0) = *reinterpret_cast<const uint4 *>(src_b);
              *reinterpret_cast<uint4 *>(&b1) = *reinterpret_cast<const uint4 *>(src_b + KC * 2);
              *reinterpret_cast<uint4 *>(&b2) = *reinterpret_cast<const uint4 *>(src_b + 2 * KC * 2);
              *reinterpret_cast<uint4 *>(&b3) = *reinterpret_cast<const uint4 *>(src_b + 3 * KC * 2);
              const uint32_t off_a = (uint32_t)row_a * 64u + (uint32_t)((v ^ ((row_a >> 1) & 3)) << 4);
              const uint32_t off_b = (uint32_t)row_b * 64u + (uint32_t)((v ^ ((row_b >> 1) & 3)) << 4);
              V8<T> o;
              o = v8_sub<T>(a0, a2); *reinterpret_cast<uint4 *>(slab + off_a) = *reinterpret_cast<const uint4 *>(&o);
              o = v8_add<T>(a1, a2); *reinterpret_cast<uint4 *>(slab + slab_bytes + off_a) = *reinterpret_cast<const uint4 *>(&o);
              o = v8_sub<T>(a2, a1); *reinterpret_cast<uint4 *>(slab + 2 * slab_bytes + off_a) = *reinterpret_cast<const uint4 *>(&o);
              o = v8_sub<T>(a1, a3); *reinterpret_cast<uint4 *>(slab + 3 * slab_bytes + off_a) = *reinterpret_cast<const uint4 *>(&o);
              o = v8_sub<T>(b0, b2); *reinterpret_cast<uint4 *>(slab + off_b) = *reinterpret_cast<const uint4 *>(&o);
              o = v8_add<T>(b1, b2); *reinterpret_cast<uint4 *>(slab + slab_bytes + off_b) = *reinterpret_cast<const uint4 *>(&o);
              o = v8_sub<T>(b2, b1); *reinterpret_cast<uint4 *>(slab + 2 * slab_bytes + off_b) = *reinterpret_cast<const uint4 *>(&o);
              o = v8_sub<T>(b1, b3); *reinterpret_cast<uint4 *>(slab + 3 * slab_bytes + off_b) = *reinterpret_cast<const uint4 *>(&o);
            }
          }
          for (int row = row_first; row < n_tasks; row += task_stride) {
            const int ir = row >> cbw_shift, cp = row - (ir << cbw_shift);
            V8<T> o0, o1, o2, o3;
            if (real && g.raw_c) {
              // the caller's few channels, gathered from the raw row into 8-channel vectors (zeros above raw_c)
              // channel ch of the stride-1 problem = element ch % raw_seg of row ch / raw_seg of the pixel's raw rows
              const T *src = reinterpret_cast<const T *>(raw) + (size_t)(ir * g.raw_fh) * g.raw_row_el + g.raw_off + (2 * cp + 3 * w) * g.raw_seg;
              __align__(16) T dv[4][8];
#pragma unroll
              for (int c = 0; c < 8; ++c) {
                const int chn = v * 8 + c;
                const int rr = chn / g.raw_seg, off = rr * g.raw_row_el + (chn - rr * g.raw_seg);
#pragma unroll
                for (int i = 0; i < 4; ++i) dv[i][c] = (chn < g.raw_c) ? src[i * g.raw_seg + off] : T(0.f);
              }
              const V8<T> d0 = *reinterpret_cast<const V8<T> *>(dv[0]), d1 = *reinterpret_cast<const V8<T> *>(dv[1]);
              const V8<T> d2 = *reinterpret_cast<const V8<T> *>(dv[2]), d3 = *reinterpret_cast<const V8<T> *>(dv[3]);
              o0 = v8_sub<T>(d0, d2); o1 = v8_add<T>(d1, d2); o2 = v8_sub<T>(d2, d1); o3 = v8_sub<T>(d1, d3);
            } else if (real) {
              const uint8_t *src = raw + ((size_t)(ir * g.patch_w + 2 * cp + 3 * w) * KC + v * 8) * 2;
              V8<T> d0, d1, d2, d3;
              *reinterpret_cast<uint4 *>(&d0) = *reinterpret_cast<const uint4 *>(src);
              *reinterpret_cast<uint4 *>(&d1) = *reinterpret_cast<const uint4 *>(src + KC * 2);
              *reinterpret_cast<uint4 *>(&d2) = *reinterpret_cast<const uint4 *>(src + 2 * KC * 2);
              *reinterpret_cast<uint4 *>(&d3) = *reinterpret_cast<const uint4 *>(src + 3 * KC * 2);
              o0 = v8_sub<T>(d0, d2); o1 = v8_add<T>(d1, d2); o2 = v8_sub<T>(d2, d1); o3 = v8_sub<T>(d1, d3);
            } else {
              const uint4 z = make_uint4(0u, 0u, 0u, 0u);
              *reinterpret_cast<uint4 *>(&o0) = z; *reinterpret_cast<uint4 *>(&o1) = z;
              *reinterpret_cast<uint4 *>(&o2) = z; *reinterpret_cast<uint4 *>(&o3) = z;
            }
            // 64-byte swizzle: 16-byte chunk index XOR ((row >> 1) & 3)
            const uint32_t off = (uint32_t)row * 64u + (uint32_t)((v ^ ((row >> 1) & 3)) << 4);
            *reinterpret_cast<uint4 *>(slab + off) = *reinterpret_cast<const uint4 *>(&o0);
            *reinterpret_cast<uint4 *>(slab + slab_bytes + off) = *reinterpret_cast<const uint4 *>(&o1);
            *reinterpret_cast<uint4 *>(slab + 2 * slab_bytes + off) = *reinterpret_cast<const uint4 *>(&o2);
            *reinterpret_cast<uint4 *>(slab + 3 * slab_bytes + off) = *reinterpret_cast<const uint4 *>(&o3);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // each writer: its stores before the MMA's reads
          __syncwarp();
          if (lane == 0) { if (PAIR) mbar_arrive_rank0(a_full(as)); else mbar_arrive(a_full(as)); }
          ++it_a;
          if (++as == sl.n_a_bufs) { as = 0; a_par ^= 1u; }
        }
        __syncwarp();
        if (alive && lane == 0) mbar_arrive(raw_empty(rs));     // all windows of this patch are transformed
        ++it_raw;
      }
    }
  } else if (warp == B_WARP) {
    // ---------------------------------------------------------------- transformed-filter slabs
    {
      bool alive = true;
      // Stages are handed over in groups of `gk` consecutive filter rows (one or all kH): one wait and one expected
      // byte count per group here, one wait and one commit per group in each MMA warp.
      const int gk = sl.b_group;
      const int n_groups = sl.n_b_stages / gk;
      int s = 0;                                    // group slot
      uint32_t s_par = 1u;                          // parity of the "group is free" wait: first round passes
      uint32_t dst = base + sl.off_b;
      ItemWalk wk = make_walk();
      for (long long item = item0; item < g.n_items && alive; item += item_step, wk.advance()) {
        const int nb = wk.nb;
        if (b_resident && item != item0) break;   // every slab of the filter is already in shared memory
        for (int kd = 0; kd < g.kD && alive; ++kd)
          for (int ch = 0; ch < g.n_chunks && alive; ++ch)
            for (int w = 0; w < g.PW && alive; ++w)
              for (int kh0 = 0; kh0 < g.kH; kh0 += gk) {
                if (!mbar_wait_warp(b_empty(s), s_par, abort_word, ERR_B_EMPTY)) { alive = false; break; }
                if (lane == 0) {
                  if (!PAIR || rank == 0)   // rank 0 of a pair expects the bytes of both halves
                    mbar_expect_tx(b_full(s), (PAIR ? 2u : 1u) * (uint32_t)(gk * sl.b_stage_bytes));
                  for (int kh = kh0; kh < kh0 + gk; ++kh) {
                    const int slab0 = ((kd * g.kH + kh) * g.PW + w) * 4;
                    if (PAIR) {             // this CTA's half (BN / 2 rows) of each slab
#pragma unroll
                      for (int j = 0; j < 4; ++j)
                        tma_load_3d_pair(dst + j * (BN / 2 * 64), &map_u, b_full(s), ch * KC,
                                         nb * BN + (int)rank * (BN / 2), slab0 + j);
                    } else {
#pragma unroll
                      for (int j = 0; j < 4; ++j)
                        tma_load_3d(dst + j * (BN * 64), &map_u, b_full(s), ch * KC, nb * BN, slab0 + j);
                    }
                    dst += (uint32_t)sl.b_stage_bytes;
                  }
                }
                dst = __shfl_sync(0xffffffffu, dst, 0);
                if (++s == n_groups) { s = 0; s_par ^= 1u; dst = base + sl.off_b; }
              }
      }
      // After an abort the filter slabs still in flight must land before the CTA may exit and free its shared memory.
      // Their bytes are counted on rank 0's barriers, which the other CTA of a pair cannot poll: a fixed delay of a
      // millisecond (a TMA load takes microseconds) covers every case.
      if (*abort_word != 0u) {
        const long long start = clock64();
        while (clock64() - start < 2000000LL) { }
      }
    }
  } else if (warp >= MMA_WARP0 && warp < MMA_WARP0 + N_MMA_THREADS) {
    // ---------------------------------------------------------------- MMA issue (rank 0 of a pair issues for both CTAs)
    // Issuing one tcgen05.mma costs the thread about as long as an N = 128 MMA runs (~60 clocks), so whatever else
    // a single issuer does (barrier waits, commits, loop branches) is time the tensor pipe idles.  Four warps, one
    // per scheduler, each issue one of the four positions of every stage (their own accumulator columns); while
    // one waits or commits the others keep the pipe fed.
    const int half = warp - MMA_WARP0;                 // position this warp issues
    if (rank == 0) {
#define MMA_WAIT(bar_, par_, aw_, code_) mbar_wait(bar_, par_, aw_, code_)   /* every lane polls; lanes differ only when a wait gives up */
#define MMA_ISSUE(d_, a_, b_, i_, acc_) do { if (PAIR) umma_f16_lohi_pair(d_, a_, b_, i_, acc_); else umma_f16_lohi(d_, a_, b_, i_, acc_); } while (0)   /* inside if (lane == 0) */
#define MMA_COMMIT(bar_) do { if (lane == 0) { if (PAIR) umma_commit_pair(bar_); else umma_commit(bar_); } } while (0)
      uint32_t n_done = 0;
      bool alive = true;
      // Everything the loop needs per stage is kept incrementally (ring position, parity, descriptor, barrier address):
      // this one thread feeds the tensor pipe, and a division or a descriptor rebuild per stage shows up as idle MMA time.
      const uint32_t slab16 = (uint32_t)(g.slab_rows * 64 / 16);
      constexpr uint32_t B_SLAB16 = (uint32_t)((PAIR ? BN / 2 : BN) * 64 / 16);   // a CTA of a pair holds half the rows
      static_assert(KC / UMMA_K == 2, "two K = 16 steps per slab");
      const int gk = sl.b_group;                          // filter rows per barrier group
      const uint32_t b_ring = (b_resident ? (uint32_t)(steps_per_item * g.PW * g.kH) : (uint32_t)sl.n_b_stages) / (uint32_t)gk;
      const uint32_t b_stage16 = (uint32_t)(sl.b_stage_bytes >> 4);
      const uint32_t b_lo_base = desc_lo(base + sl.off_b);
      uint32_t bs = 0, b_par = 0, b_lo0 = b_lo_base;
      const uint32_t n_a = (uint32_t)sl.n_a_bufs;
      const uint32_t a_lo_buf0 = desc_lo(base + sl.off_a[0]), a_lo_buf1 = desc_lo(base + sl.off_a[1]), a_lo_buf2 = desc_lo(base + sl.off_a[2]);
      uint32_t as = 0, a_par = 0;
      const uint32_t kh_step16 = (uint32_t)(g.CBW * 4);    // one filter row further = CBW slab rows of 64 bytes
      const int tail_chunk = (g.Cp - (g.n_chunks - 1) * KC > UMMA_K) ? -1 : g.n_chunks - 1;   // chunk with one K step only
      const int kH = g.kH, PW = g.PW, n_chunks = g.n_chunks;   // loop bounds in registers
      const long long n_items = g.n_items;
      const uint32_t a_half16 = (uint32_t)half * slab16, b_half16 = (uint32_t)half * B_SLAB16;
      for (long long item = item0; item < n_items && alive; item += item_step, ++n_done) {
        const int ab = (ACC_BUFS == 2) ? (int)(n_done & 1u) : 0;
        const uint32_t use = (ACC_BUFS == 2) ? (n_done >> 1) : n_done;
        if (!MMA_WAIT(acc_empty(ab), (use & 1u) ^ 1u, abort_word, ERR_MMA_ACC)) { alive = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem_base + (uint32_t)(ab * ACC_COLS);
        uint32_t acc0 = 0u;
        int ch = 0;
        if (b_resident) { bs = 0; b_lo0 = b_lo_base; }      // a resident filter: every item starts at its first stage
        for (int step = 0; step < steps_per_item && alive; ++step) {
          // a slab with at most 16 real channels (few-channel input, or the tail of C) needs one K = 16 step only
          const bool k2 = ch != tail_chunk;
          if (++ch == n_chunks) ch = 0;
          for (int w = 0; w < PW && alive; ++w) {
            if (!MMA_WAIT(a_full((int)as), a_par, abort_word, ERR_MMA_A)) { alive = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t a_lo_kh = (as == 0 ? a_lo_buf0 : (as == 1 ? a_lo_buf1 : a_lo_buf2)) + a_half16;
            // one group = gk filter rows behind one full / empty barrier pair: one wait, 2 gk MMAs back to back, one commit.
            // Straight-line code for the usual three rows (a taken branch costs this lone warp ~100 clocks of
            // instruction fetch); whatever this warp does besides issuing is time its position's MMAs are not queued.
            auto issue_row = [&]() {
              if (lane == 0) {
#pragma unroll
                for (int mb = 0; mb < MB; ++mb) {
                  const uint32_t a_lo = a_lo_kh + (uint32_t)(mb * BM * 4);      // block mb starts RB * CBW = 128 rows later
                  const uint32_t b_lo = b_lo0 + b_half16;
                  const uint32_t d_col = acc + (uint32_t)((mb * 4 + half) * BN);
                  MMA_ISSUE(d_col, a_lo, b_lo, idesc, acc0);
                  if (k2) MMA_ISSUE(d_col, a_lo + 2u, b_lo + 2u, idesc, 1u);     // second K = 16 step: 32 bytes further
                }
              }
              acc0 = 1u;
              a_lo_kh += kh_step16;
              b_lo0 += b_stage16;
            };
            auto group_begin = [&]() -> bool {
              if (!(b_resident && n_done > 0))
                if (!mbar_wait(b_full((int)bs), b_par, abort_word, ERR_MMA_B)) return false;
              return true;
            };
            auto group_end = [&]() {
              if (!b_resident) MMA_COMMIT(b_empty((int)bs));
              if (++bs == b_ring) { bs = 0; b_lo0 = b_lo_base; b_par = b_resident ? 0u : (b_par ^ 1u); }
            };
            if (b_resident && n_done > 0) {
              // The whole filter sits in shared memory and has landed: no barrier, no ring bookkeeping -- the rows of an
              // item are consecutive stages.  These warps run alone on code nothing else keeps in the instruction
              // cache (~10 clocks an instruction, measured): with one or two MMAs per row the row's bookkeeping, not
              // the tensor pipe, set the pace of the few-channel and K = 64 layers.
              if (kH == 3) { issue_row(); issue_row(); issue_row(); }
              else for (int kh = 0; kh < kH; ++kh) issue_row();
            } else if (gk == 3) {          // kH == 3, all three rows in one group
              if (!group_begin()) { alive = false; break; }
              issue_row(); issue_row(); issue_row();
              group_end();
            } else if (kH == 3) {   // gk == 1
              bool ok = group_begin();
              if (ok) { issue_row(); group_end(); ok = group_begin(); }
              if (ok) { issue_row(); group_end(); ok = group_begin(); }
              if (ok) { issue_row(); group_end(); }
              if (!ok) { alive = false; break; }
            } else {                // any other height: single-row groups (gk == 1), one short loop body
              for (int kh = 0; kh < kH && alive; ++kh) {
                alive = group_begin();
                if (alive) { issue_row(); group_end(); }
              }
              if (!alive) break;
            }
            MMA_COMMIT(a_empty((int)as));
            if (++as == n_a) { as = 0; a_par ^= 1u; }
          }
        }
        MMA_COMMIT(acc_full(ab));
      }
#undef MMA_WAIT
#undef MMA_ISSUE
#undef MMA_COMMIT
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    // Eight warps: warp w reads TMEM lane quarter w & 3 (a hardware rule) and one half of the accumulator columns.
    const int qd = warp & 3;                           // TMEM lane quarter
    const int chalf = (warp - EPI_WARP0) >> 2;         // which half of the BN columns
    const int row = qd * 32 + lane;                    // tile of the block: (out row, column pair)
    const int cbw_shift = g.CBW == 16 ? 4 : 3;
    const int tr = row >> cbw_shift, tcp = row - (tr << cbw_shift);
    const bool relu = (g.epilogue & WINOCONV_EPI_RELU) != 0;
    const bool has_bias = (g.epilogue & WINOCONV_EPI_BIAS) != 0;
    const bool pool = (g.epilogue & WINOCONV_EPI_POOL2) != 0;
    // widest store the output allows: 32 bytes (K % 16, 32-byte aligned base), 16 bytes (K % 8), or elements
    const int st_mode = ((g.K % 16) == 0 && (reinterpret_cast<uintptr_t>(y) & 31u) == 0) ? 2 : ((g.K % 8) == 0 ? 1 : 0);
    const int K = g.K;
    constexpr int C_PER_WARP = BN / 2;
    uint32_t n_done = 0;
    bool alive = true;
    ItemWalk wk = make_walk();
    for (long long item = item0; item < g.n_items && alive; item += item_step, ++n_done, wk.advance()) {
      const int n = PAIR ? 2 * wk.n5 + (int)rank : wk.n5, od = wk.od, rb = wk.rb, cb = wk.cb, nb = wk.nb;
      const int ab = (ACC_BUFS == 2) ? (int)(n_done & 1u) : 0;
      const uint32_t use = (ACC_BUFS == 2) ? (n_done >> 1) : n_done;
      unsigned got = 0;
      if (lane == 0) got = mbar_wait(acc_full(ab), use & 1u, abort_word, ERR_EPI) ? 1u : 0u;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (got == 0u) { alive = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int ow = (cb * g.CBW + tcp) * 2;
      const int k0 = nb * BN + chalf * C_PER_WARP;      // first output channel of this warp
#pragma unroll 1
      for (int mb = 0; mb < MB; ++mb) {
        const uint32_t t_lane = tmem_base + ((uint32_t)(qd * 32) << 16) + (uint32_t)(ab * ACC_COLS + mb * 4 * BN + chalf * C_PER_WARP);
        const int oh = (rb * MB + mb) * g.RB + tr;
        // destination of this thread's tile, and which of its stores are inside the output
        T *dst;
        bool st0, st1;
        if (pool) {
          const int ph = oh >> 1, pw = ow >> 1;
          dst = y + ((((long long)n * g.oD + od) * g.yH + ph) * g.yW + pw) * K + k0;
          st0 = (tr & 1) == 0 && ph < g.yH && pw < g.yW && n < g.N;
          st1 = false;
        } else {
          dst = y + ((((long long)n * g.oD + od) * g.oH + oh) * g.oW + ow) * K + k0;
          const bool in = oh < g.oH && n < g.N;
          st0 = in && ow < g.oW;
          st1 = in && ow + 1 < g.oW;
        }
        uint32_t p0[8], p1[8], p2[8], p3[8];
#pragma unroll 1
        for (int c0 = 0; c0 < C_PER_WARP; c0 += 16) {
          uint32_t pk0[8], pk1[8];                     // 16 channels of the two output pixels, packed
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int cc = c0 + 8 * h;
            tmem_ld_x8(t_lane + (uint32_t)(0 * BN + cc), p0);
            tmem_ld_x8(t_lane + (uint32_t)(1 * BN + cc), p1);
            tmem_ld_x8(t_lane + (uint32_t)(2 * BN + cc), p2);
            tmem_ld_x8(t_lane + (uint32_t)(3 * BN + cc), p3);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (h == 1 && c0 + 16 >= C_PER_WARP && mb == MB - 1) {   // last columns are in registers: hand the accumulator back
              asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
              __syncwarp();
              if (lane == 0) { if (PAIR) mbar_arrive_rank0(acc_empty(ab)); else mbar_arrive(acc_empty(ab)); }
            }
            const int kbase = k0 + cc;
            // A^T along W on channel pairs with the packed fp32 adds of sm_100 (y0 = a0 + a1 + a2, y1 = a1 - a2 - a3), one
            // rounding to the 16-bit pair, then ReLU and the pool's maxima on the packed halves: rounding is monotonic,
            // so max-then-round and round-then-max give the same bits at half the instructions.
            uint32_t v0[4], v1[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const uint64_t a0 = pack_f32x2(p0[2 * c], p0[2 * c + 1]), a1 = pack_f32x2(p1[2 * c], p1[2 * c + 1]);
              const uint64_t a2 = pack_f32x2(p2[2 * c], p2[2 * c + 1]), a3 = pack_f32x2(p3[2 * c], p3[2 * c + 1]);
              uint64_t y0 = add_f32x2(add_f32x2(a0, a1), a2);
              uint64_t y1 = sub_f32x2(sub_f32x2(a1, a2), a3);
              if (has_bias) {
                const float b_lo = (kbase + 2 * c < K) ? Elem<T>::load(bias + kbase + 2 * c) : 0.f;
                const float b_hi = (kbase + 2 * c + 1 < K) ? Elem<T>::load(bias + kbase + 2 * c + 1) : 0.f;
                const uint64_t bv = pack_f32x2(__float_as_uint(b_lo), __float_as_uint(b_hi));
                y0 = add_f32x2(y0, bv);
                y1 = add_f32x2(y1, bv);
              }
              v0[c] = P2<T>::round_pair(y0);
              v1[c] = P2<T>::round_pair(y1);
            }
            if (pool) {
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                uint32_t mx = P2<T>::max2(v0[c], v1[c]);
                mx = P2<T>::max2(mx, __shfl_xor_sync(0xffffffffu, mx, g.CBW));   // the other output row of the 2x2 window
                v0[c] = relu ? P2<T>::max2(mx, 0u) : mx;
              }
            } else if (relu) {
#pragma unroll
              for (int c = 0; c < 4; ++c) { v0[c] = P2<T>::max2(v0[c], 0u); v1[c] = P2<T>::max2(v1[c], 0u); }
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) { pk0[4 * h + c] = v0[c]; pk1[4 * h + c] = v1[c]; }
          }
          const int kb16 = k0 + c0;
          if (kb16 < K) {
            if (st0) store16p<T>(dst + c0, pk0, kb16, K, st_mode);
            if (st1) store16p<T>(dst + K + c0, pk1, kb16, K, st_mode);
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (PAIR) cluster_sync_all();   // neither CTA frees tensor memory or exits while the other may still use it
  if (warp == MMA_WARP0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// U[slab][k][c], slab = ((kd * kH + kh) * PW + w) * 4 + j:  G (3 taps of window w, zero padded) along W.
// With phases (stride 2 folded into channels) channel c = phase * C0 + c0 and tap (kd, kh, kw) of the stride-1 kernel is
// tap (fD * kd + phase_d, fH * kh + phase_h, fW * kw + phase_w) of the caller's kernel (zero beyond its extent).
struct FilterPhases {
  int on, fD, fH, fW, C0, kD0, kH0, kW0;
  int Cs;     // channel stride between polyphase parts in the phase-channel order (C0, or C0 rounded up to 32)
};
template <typename T>
__global__ void __launch_bounds__(256) rowfused_filter_kernel(const T *__restrict__ wgt, T *__restrict__ u, int C, int Cp,
                                                              int K, int kD, int kH, int kW, int PW, int layout,
                                                              FilterPhases ph) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long per_k = (long long)kD * kH * PW * Cp;
  if (idx >= per_k * K) return;
  const int k = (int)(idx / per_k);
  long long rem = idx - (long long)k * per_k;
  const int c = (int)(rem % Cp); rem /= Cp;
  const int w = (int)(rem % PW); rem /= PW;
  const int kh = (int)(rem % kH);
  const int kd = (int)(rem / kH);
  float a[3] = {0.f, 0.f, 0.f}, o[4];
  // the caller's channel and kernel extents, and this element's phase offsets
  int c0 = c, C0 = C, eD = kD, eH = kH, eW = kW, fD = 1, fH = 1, fW = 1, pd = 0, phh = 0, pw = 0;
  bool valid = c < C;
  if (ph.on) {
    C0 = ph.C0; eD = ph.kD0; eH = ph.kH0; eW = ph.kW0; fD = ph.fD; fH = ph.fH; fW = ph.fW;
    int phase = c / ph.Cs;
    c0 = c - phase * ph.Cs;
    valid = phase < fD * fH * fW && c0 < C0;
    pw = phase % fW; phase /= fW;
    phh = phase % fH; phase /= fH;
    pd = phase;
  }
  if (valid) {
    const int td = fD * kd + pd, th = fH * kh + phh;
#pragma unroll
    for (int t = 0; t < 3; ++t) {
      const int kw = 3 * w + t;
      const int tw = fW * kw + pw;
      if (kw < kW && td < eD && th < eH && tw < eW) {
        const long long off = layout == WINOCONV_W_KCRS ? ((((long long)k * C0 + c0) * eD + td) * eH + th) * eW + tw
                                                        : ((((long long)td * eH + th) * eW + tw) * C0 + c0) * K + k;
        a[t] = Elem<T>::load(wgt + off);
      }
    }
  }
  Xf<2, 3>::g<1, 1>(a, o);
  const long long slab0 = (((long long)kd * kH + kh) * PW + w) * 4;
#pragma unroll
  for (int j = 0; j < 4; ++j) Elem<T>::store(u + ((slab0 + j) * K + k) * Cp + c, o[j]);
}

// zero-pads the channel dimension to a multiple of 8 so the input can be addressed by TMA; one thread writes one
// 16-byte group of eight channels
template <typename T>
__global__ void __launch_bounds__(256) pad_channels_kernel(const T *__restrict__ x, T *__restrict__ xp, long long pixels,
                                                           int C, int Cp) {
  const int groups = Cp / 8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= pixels * groups) return;
  const long long px = idx / groups;
  const int c0 = (int)(idx - px * groups) * 8;
  __align__(16) T v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = (c0 + i < C) ? x[px * C + c0 + i] : T(0.f);
  *reinterpret_cast<uint4 *>(xp + px * Cp + c0) = *reinterpret_cast<const uint4 *>(v);
}

// Stride 2 -> stride 1: xs[n][id][ih][iw][phase * C0 + c] = x_padded[n][fD * id + pd][fH * ih + ph][fW * iw + pw][c]
// (zero outside the caller's tensor and in the channels that pad phases * C0 to a multiple of 8).  One thread writes
// one 16-byte group of eight channels.
struct PhaseGeom {
  int N, D, H, W, Cp;          // destination extents (stride-1 problem)
  int fD, fH, fW, C0, D0, H0, W0, pD0, pH0, pW0;
};
template <typename T>
__global__ void __launch_bounds__(256) phases_to_channels_kernel(const T *__restrict__ x, T *__restrict__ xs, PhaseGeom q) {
  const unsigned groups = (unsigned)(q.Cp / 8);
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long pixels = (long long)q.N * q.D * q.H * q.W;
  if (idx >= pixels * groups) return;
  const long long px = idx / groups;
  const int cg = (int)(idx - px * groups) * 8;
  // pixel coordinates: one 64-bit division by the row length, the rest in 32 bits
  const long long row = px / q.W;
  const int iw = (int)(px - row * q.W);
  const unsigned rowu = (unsigned)row;                  // N * D * H rows: fits 32 bits for any tensor that fits memory
  const unsigned ndh = rowu / (unsigned)q.H;
  const int ih = (int)(rowu - ndh * (unsigned)q.H);
  const int n = (int)(ndh / (unsigned)q.D);
  const int id = (int)(ndh - (unsigned)n * (unsigned)q.D);
  const int C = q.fD * q.fH * q.fW * q.C0;
  // channel c = phase * C0 + c0 is walked incrementally: one division for the first channel of the group
  int phase = cg / q.C0, c0 = cg - phase * q.C0;
  const T *src = nullptr;                                // first channel of the current phase's source pixel, or null
  bool fresh = true;
  __align__(16) T v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    T val = T(0.f);
    if (cg + i < C) {
      if (fresh) {
        const int pw = phase % q.fW, t = phase / q.fW;
        const int ph = t % q.fH, pd = t / q.fH;
        const int sd = q.fD * id + pd - q.pD0, sh = q.fH * ih + ph - q.pH0, sw = q.fW * iw + pw - q.pW0;
        src = (sd >= 0 && sd < q.D0 && sh >= 0 && sh < q.H0 && sw >= 0 && sw < q.W0)
                  ? x + ((((long long)n * q.D0 + sd) * q.H0 + sh) * q.W0 + sw) * q.C0
                  : nullptr;
        fresh = false;
      }
      if (src) val = src[c0];
      if (++c0 == q.C0) { c0 = 0; ++phase; fresh = true; }
    }
    v[i] = val;
  }
  *reinterpret_cast<uint4 *>(xs + idx * 8) = *reinterpret_cast<const uint4 *>(v);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void *p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

}  // namespace rowf

// Fills the geometry of the row-piece kernel for the stride-1 problem in `d` (a stride-2 convolution arrives here
// already folded into phase channels); returns false when it does not apply (a patch / slab set that does not fit
// shared memory).
bool rowfused_plan(const RowDesc &d, RowPlan *out) {
  using namespace rowf;
  if (d.sD != 1 || d.sH != 1 || d.sW != 1) return false;
  if (d.kH > 10 || d.kW > 10 || d.kD > 10) return false;   // taller kernels: the planner below decides whether patch and slabs fit
  RowPlan p;
  int Cp = (d.C + 7) / 8 * 8;
  p.Cp = Cp;
  p.PW = (d.kW + 2) / 3;
  // Work item: MB tile blocks stacked along H x BN output channels, MB * BN <= 128 (the 512 TMEM columns hold
  // MB x 4 positions x BN).  One block x 128 channels is the default.  Two blocks x 64 channels halve the filter
  // bytes streamed per multiply-add but were measured slower on B200 (VGG-16: 17.3 vs 11.9 ms): an N = 64 MMA
  // takes as long as an N = 128 one, and two blocks leave room for only one slab buffer.  WINOCONV_ROW_MB=2
  // selects them for experiments.
  const int ncp = (d.oW + 1) / 2;
  auto padded = [&](int rows_item, int cbw) {
    return (long long)((d.oH + rows_item - 1) / rows_item) * rows_item * ((ncp + cbw - 1) / cbw) * cbw;
  };
  static const int forced_mb = [] { const char *v = getenv("WINOCONV_ROW_MB"); return v && *v ? atoi(v) : 0; }();
  const int best_mb = forced_mb == 2 ? 2 : 1;
  const int best_cbw = padded(best_mb * 8, 16) <= padded(best_mb * 16, 8) ? 16 : 8;
  p.MB = best_mb;
  p.BN = (p.MB == 2 || d.K <= 64) ? 64 : 128;
  p.CBW = best_cbw;
  p.RB = 128 / p.CBW;
  p.n_rb = (d.oH + p.MB * p.RB - 1) / (p.MB * p.RB);
  p.n_cb = (ncp + p.CBW - 1) / p.CBW;
  p.slab_rows = (p.MB * p.RB + d.kH - 1) * p.CBW;
  p.patch_h = p.MB * p.RB + d.kH - 1;
  p.patch_w = 2 * p.CBW + 3 * p.PW - 1;
  p.n_chunks = (Cp + KC - 1) / KC;
  p.n_nblocks = (d.K + p.BN - 1) / p.BN;
  p.slabs = d.kD * d.kH * p.PW * 4;
  p.filter_elems = (long long)p.slabs * d.K * Cp;
  // CTA pairs: the two SMs of a cluster take images 2n and 2n + 1 of one item and share every filter slab (each loads
  // half of it).  One M = 256 MMA then covers both tile blocks in the time of an M = 128 one whenever the instruction
  // floor (~60 clocks) binds, i.e. at N = 64 it doubles the MMA rate; at N = 128 it halves the filter bytes an SM
  // pulls per multiply-add and leaves room for twice as many stages.  Used whenever the batch has two images.
  static const int pair_env = [] { const char *v = getenv("WINOCONV_ROW_PAIR"); return v && *v ? atoi(v) : -1; }();
  p.pair = (pair_env != 0 && p.MB == 1 && d.N >= 2) ? 1 : 0;
  p.n_items = (long long)(p.pair ? (d.N + 1) / 2 : d.N) * d.oD * p.n_rb * p.n_cb * p.n_nblocks;
  if (p.patch_w > 256 || p.patch_h > 256) return false;
  // Fewer than eight channels (RGB): TMA wants 16-byte pixels, but a row of W * C elements is a legal innermost
  // dimension when W * C is a multiple of eight, and a block's first pixel then always lies the same number of elements
  // past a multiple of eight (a block is 16 or 32 pixels wide).  The producers gather the few channels into 8-channel
  // vectors as they transform, so no padded copy of x is made.  WINOCONV_ROW_RAWC=0 keeps the padding pass.
  static const int rawc_env = [] { const char *v = getenv("WINOCONV_ROW_RAWC"); return v && *v ? atoi(v) : 1; }();
  p.raw_c = 0; p.raw_off = 0; p.raw_row_el = 0;
  p.raw_seg = 0; p.raw_fh = 1; p.raw_pd = 0; p.raw_ph = 0; p.raw_pw = 0;
  if (d.phases <= 1 && d.C < 8 && ((long long)d.W * d.C) % 8 == 0 && rawc_env != 0) {
    const int off = ((-(d.pW * d.C)) % 8 + 8) % 8;
    const int row_el = (off + p.patch_w * d.C + 7) / 8 * 8;
    if (row_el <= 256) {
      p.raw_c = d.C; p.raw_off = off; p.raw_row_el = row_el;
      p.raw_seg = d.C; p.raw_fh = 1; p.raw_pd = d.pD; p.raw_ph = d.pH; p.raw_pw = d.pW * d.C;
    }
  }
  // Stride 2 in H and / or W over few channels (a 7x7 stride-2 RGB stem: 4 phases x 3 = 12 channels): the phase channels
  // of a pixel of the stride-1 problem are fW * C0 consecutive elements in each of fH consecutive rows of x, so the same
  // raw-row patch serves and neither the phase-gathered copy of x nor its scratch is needed.
  if (d.phases > 1 && d.fD == 1 && d.C <= 32 && ((long long)d.W0 * d.C0) % 8 == 0 && rawc_env != 0) {
    const int seg = d.fW * d.C0;
    const int off = ((-(d.pW0 * d.C0)) % 8 + 8) % 8;
    const int row_el = (off + p.patch_w * seg + 7) / 8 * 8;
    if (row_el <= 256 && p.patch_h * d.fH <= 256 && (2 * p.CBW * seg) % 8 == 0) {
      p.raw_c = d.C; p.raw_off = off; p.raw_row_el = row_el;
      p.raw_seg = seg; p.raw_fh = d.fH; p.raw_pd = d.pD0; p.raw_ph = d.pH0; p.raw_pw = d.pW0 * d.C0;
    }
  }
  // Stride 2 in H and / or W over a multiple of 32 channels: every 32-channel step of the stride-1 problem is one
  // polyphase part of the caller's tensor, which a tensor map with element strides (fW, fH) loads directly.
  p.s2_chunks = 0;
  // A channel count that is a multiple of 8 but not of 32 gets its polyphase parts 32-aligned in the phase-channel
  // order (the map's zero fill and zero filter channels pad each part).
  // Taken while the padding adds at most a third to the reduction.
  const int s2_padded_chunks = d.phases * ((d.C0 + KC - 1) / KC);
  if (d.phases > 1 && !p.raw_c && d.fD == 1 && d.C0 % 8 == 0 && d.fW * p.patch_w <= 256 && d.fH * p.patch_h <= 256 &&
      3 * s2_padded_chunks <= 4 * p.n_chunks && rawc_env != 0) {
    p.s2_chunks = (d.C0 + KC - 1) / KC;
    Cp = d.phases * p.s2_chunks * KC;
    p.Cp = Cp;
    p.n_chunks = Cp / KC;
    p.filter_elems = (long long)p.slabs * d.K * Cp;
  }
  // shared memory: 2 raw patches, 2 slab sets (1 if two do not leave room for 3 filter stages), then as many
  // filter stages as fit (2..8)
  const int raw_box_bytes = p.raw_c ? p.patch_h * p.raw_fh * p.raw_row_el * 2 : p.patch_h * p.patch_w * KC * 2;
  const int raw_bytes = ((raw_box_bytes + 127) / 128) * 128;
  const int a_bytes = ((4 * p.slab_rows * 64 + 1023) / 1024) * 1024;
  const int b_stage = 4 * (p.pair ? p.BN / 2 : p.BN) * 64;
  const int budget = 227 * 1024;
  // three slab sets when three filter stages still fit beside them (CTA pairs: half-size stages): the producers then
  // run a full 32-channel step ahead of the MMAs instead of racing the step in flight (measured on the 256- and
  // 512-channel VGG layers: 0.65 ms against 0.69 ms with two sets and eight stages)
  static const int na_env = [] { const char *v = getenv("WINOCONV_ROW_ABUFS"); return v && *v ? atoi(v) : 0; }();
  int n_a = (na_env >= 1 && na_env <= 3) ? na_env : 3;
  int fixed = 2 * raw_bytes + n_a * a_bytes + 1024 /*bars*/ + 1024 /*align*/;
  static const int minb_env = [] { const char *v = getenv("WINOCONV_ROW_MINB"); return v && *v ? atoi(v) : 3; }();
  if (n_a == 3 && (budget - fixed) / b_stage < minb_env) {
    n_a = 2;
    fixed = 2 * raw_bytes + n_a * a_bytes + 2048;
  }
  if (n_a == 2 && (budget - fixed) / b_stage < 3) {
    n_a = 1;
    fixed = 2 * raw_bytes + n_a * a_bytes + 2048;
  }
  int nb = (budget - fixed) / b_stage;
  // One channel block whose whole item's filter slabs would fit the ring if a slab set gave up its room: keeping the
  // filter resident (loaded once per CTA) beats the third slab set (a 7x7 stride-2 layer run as 4x4 over 12
  // channels has 8 stages per item: four fit beside three slab sets, eight beside two).
  const int stages_per_item = p.n_chunks * d.kD * d.kH * p.PW;
  if (p.n_nblocks == 1 && n_a == 3 && nb < stages_per_item && stages_per_item <= 8) {
    const int fixed2 = 2 * raw_bytes + 2 * a_bytes + 2048;
    if ((budget - fixed2) / b_stage >= stages_per_item) {
      n_a = 2;
      fixed = fixed2;
      nb = (budget - fixed) / b_stage;
    }
  }
  if (nb < 2) return false;
  if (nb > 8) nb = 8;
  // Streamed 3-row kernels: hand the filter over in groups of all three rows (one barrier round trip per 32-channel
  // step and MMA warp instead of three) when two such groups fit the ring, giving up the third slab set if that is
  // what it takes.  WINOCONV_ROW_BGROUP=1 keeps single-row stages.
  static const int bgroup_env = [] { const char *v = getenv("WINOCONV_ROW_BGROUP"); return v && *v ? atoi(v) : 0; }();
  p.b_group = 1;
  const bool resident = p.n_nblocks == 1 && stages_per_item <= nb;
  if (d.kH == 3 && !resident && bgroup_env != 1) {
    int n_a_g = n_a;
    int room = (budget - (2 * raw_bytes + n_a_g * a_bytes + 2048)) / b_stage;
    if (room < 6 && n_a_g == 3) { n_a_g = 2; room = (budget - (2 * raw_bytes + n_a_g * a_bytes + 2048)) / b_stage; }
    if (room >= 6) {
      p.b_group = 3;
      n_a = n_a_g;
      fixed = 2 * raw_bytes + n_a * a_bytes + 2048;
      nb = 6;
    }
  }
  p.n_a_bufs = n_a;
  p.raw_bytes = raw_bytes; p.a_bytes = a_bytes; p.b_stage_bytes = b_stage; p.n_b_stages = nb;
  p.smem_total = fixed + nb * b_stage;
  *out = p;
  return true;
}

cudaError_t launch_rowfused_filter_transform(const RowDesc &d, const RowPlan &p, int dtype, const void *w, void *u, cudaStream_t s) {
  const long long n = (long long)d.kD * d.kH * p.PW * p.Cp * d.K;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  rowf::FilterPhases ph = {};
  if (d.phases > 1) {
    ph.on = 1; ph.fD = d.fD; ph.fH = d.fH; ph.fW = d.fW; ph.C0 = d.C0; ph.kD0 = d.kD0; ph.kH0 = d.kH0; ph.kW0 = d.kW0;
    ph.Cs = p.s2_chunks ? p.s2_chunks * rowf::KC : d.C0;
  }
  if (dtype == WINOCONV_F16)
    rowf::rowfused_filter_kernel<__half><<<blocks, 256, 0, s>>>((const __half *)w, (__half *)u, d.C, p.Cp, d.K, d.kD, d.kH, d.kW, p.PW, d.weight_layout, ph);
  else
    rowf::rowfused_filter_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16 *)w, (__nv_bfloat16 *)u, d.C, p.Cp, d.K, d.kD, d.kH, d.kW, p.PW, d.weight_layout, ph);
  return cudaGetLastError();
}

template <typename T, int BN, int MB, bool PAIR>
static cudaError_t launch_rf(const RowDesc &d, const RowPlan &p, const CUtensorMap &mx, const CUtensorMap &mu, void *y,
                             const void *bias, int sm_count, uint32_t idesc, cudaStream_t s, const char **detail) {
  using namespace rowf;
  auto kern = rowfused_kernel<T, BN, MB, PAIR>;
  // Per device and kernel instance, remembered across calls (an eager caller pays these host calls per layer):
  // the largest dynamic shared memory size set so far, and how many CTA pairs can be resident at once.
  static std::mutex cache_mutex;
  static std::map<int, std::pair<int, int>> cache;   // device -> (smem attribute set, resident clusters or 0)
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { *detail = "cudaGetDevice failed"; return e; }
  int known_clusters = 0;
  {
    std::lock_guard<std::mutex> lock(cache_mutex);
    std::pair<int, int> &c = cache[dev];
    if (c.first < p.smem_total) {
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, p.smem_total);
      if (e != cudaSuccess) { *detail = "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed"; return e; }
      c.first = p.smem_total;
    }
    known_clusters = c.second;
  }
  RGeom g;
  g.N = d.N; g.C = d.C; g.K = d.K; g.Cp = p.Cp; g.D = d.D; g.H = d.H; g.W = d.W; g.oD = d.oD; g.oH = d.oH; g.oW = d.oW;
  g.yH = d.yH; g.yW = d.yW; g.pD = d.pD; g.pH = d.pH; g.pW = d.pW; g.kD = d.kD; g.kH = d.kH; g.kW = d.kW;
  g.PW = p.PW; g.RB = p.RB; g.CBW = p.CBW; g.MB = p.MB; g.n_rb = p.n_rb; g.n_cb = p.n_cb; g.slab_rows = p.slab_rows;
  g.patch_h = p.patch_h; g.patch_w = p.patch_w; g.n_chunks = p.n_chunks; g.n_nblocks = p.n_nblocks;
  g.n_items = p.n_items; g.epilogue = d.epilogue;
  g.raw_c = p.raw_c; g.raw_off = p.raw_off; g.raw_row_el = p.raw_row_el;
  g.s2_chunks = p.s2_chunks; g.s2_fh = d.fH; g.s2_fw = d.fW; g.s2_pd = d.pD0; g.s2_ph = d.pH0; g.s2_pw = d.pW0;
  g.raw_seg = p.raw_seg; g.raw_fh = p.raw_fh; g.raw_pd = p.raw_pd; g.raw_ph = p.raw_ph; g.raw_pw = p.raw_pw;
  Smem sl;
  sl.raw_bytes = p.raw_c ? p.patch_h * p.raw_fh * p.raw_row_el * 2 : p.patch_h * p.patch_w * KC * 2;   // bytes the TMA box delivers
  sl.a_bytes = p.a_bytes; sl.b_stage_bytes = p.b_stage_bytes; sl.n_b_stages = p.n_b_stages;
  sl.n_a_bufs = p.n_a_bufs;
  sl.b_group = p.b_group;
  sl.off_a[0] = 0;                                                 // slabs first: 1024-byte aligned
  sl.off_a[1] = p.n_a_bufs >= 2 ? p.a_bytes : 0;
  sl.off_a[2] = p.n_a_bufs >= 3 ? 2 * p.a_bytes : 0;
  sl.off_b = p.n_a_bufs * p.a_bytes;                               // filter stages: multiples of 1024
  sl.off_raw[0] = sl.off_b + p.n_b_stages * p.b_stage_bytes;
  sl.off_raw[1] = sl.off_raw[0] + p.raw_bytes;
  sl.off_bars = sl.off_raw[1] + p.raw_bytes;
  sl.total = p.smem_total;
  if (PAIR) {
    const int pairs = (int)std::min<long long>(p.n_items, sm_count / 2);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
    cfg.blockDim = dim3(N_THREADS, 1, 1);
    cfg.dynamicSmemBytes = (size_t)p.smem_total;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // one resident pair per two SMs where the GPCs allow it; fewer pairs when they do not (the items are strided over
    // the pairs launched, so every launched pair must be resident)
    int max_clusters = known_clusters;
    if (max_clusters == 0 && cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) == cudaSuccess && max_clusters > 0) {
      std::lock_guard<std::mutex> lock(cache_mutex);
      cache[dev].second = max_clusters;
    }
    if (max_clusters > 0 && max_clusters < pairs) cfg.gridDim = dim3((unsigned)(2 * max_clusters), 1, 1);
    return cudaLaunchKernelEx(&cfg, kern, mx, mu, (T *)y, (const T *)bias, g, sl, idesc);
  }
  const int grid = (int)std::min<long long>(p.n_items, sm_count);
  kern<<<grid, N_THREADS, p.smem_total, s>>>(mx, mu, (T *)y, (const T *)bias, g, sl, idesc);
  return cudaGetLastError();
}

cudaError_t launch_rowfused_forward(const RowDesc &d, const RowPlan &p, int dtype, const void *x, const void *u,
                                    const void *bias, void *y, void *pad_ws, cudaStream_t s, const char **detail) {
  using namespace rowf;
  *detail = "";
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) { *detail = "cuTensorMapEncodeTiled unavailable"; return cudaErrorNotSupported; }
  const void *xin = x;
  if (d.phases > 1 && !p.raw_c && !p.s2_chunks) {   // stride 2: gather the polyphase parts into channels (and pad them to a multiple of 8)
    if (!pad_ws) { *detail = "phase-gather scratch missing"; return cudaErrorInvalidValue; }
    PhaseGeom q;
    q.N = d.N; q.D = d.D; q.H = d.H; q.W = d.W; q.Cp = p.Cp;
    q.fD = d.fD; q.fH = d.fH; q.fW = d.fW; q.C0 = d.C0; q.D0 = d.D0; q.H0 = d.H0; q.W0 = d.W0;
    q.pD0 = d.pD0; q.pH0 = d.pH0; q.pW0 = d.pW0;
    const long long groups = (long long)d.N * d.D * d.H * d.W * (p.Cp / 8);
    const unsigned blocks = (unsigned)((groups + 255) / 256);
    if (dtype == WINOCONV_F16)
      phases_to_channels_kernel<__half><<<blocks, 256, 0, s>>>((const __half *)x, (__half *)pad_ws, q);
    else
      phases_to_channels_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16 *)x, (__nv_bfloat16 *)pad_ws, q);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { *detail = "phase gather launch failed"; return e; }
    xin = pad_ws;
  } else if (p.Cp != d.C && !p.raw_c && !p.s2_chunks) {   // channels not a multiple of 8: TMA needs 16-byte pixel strides, so pad into scratch first
    if (!pad_ws) { *detail = "channel padding scratch missing"; return cudaErrorInvalidValue; }
    const long long pixels = (long long)d.N * d.D * d.H * d.W;
    const unsigned blocks = (unsigned)((pixels * (p.Cp / 8) + 255) / 256);
    if (dtype == WINOCONV_F16)
      pad_channels_kernel<__half><<<blocks, 256, 0, s>>>((const __half *)x, (__half *)pad_ws, pixels, d.C, p.Cp);
    else
      pad_channels_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16 *)x, (__nv_bfloat16 *)pad_ws, pixels, d.C, p.Cp);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { *detail = "channel padding launch failed"; return e; }
    xin = pad_ws;
  }
  const CUtensorMapDataType dt = dtype == WINOCONV_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap mx, mu;
  if (p.raw_c) {   // x as it lies: [N, D, H, W * C] (the caller's tensor, also for a stride-2 layer)
    const bool ph = d.phases > 1;
    const cuuint64_t row = ph ? (cuuint64_t)d.W0 * d.C0 : (cuuint64_t)d.W * d.C;
    const cuuint64_t hh = ph ? (cuuint64_t)d.H0 : (cuuint64_t)d.H, dd = ph ? (cuuint64_t)d.D0 : (cuuint64_t)d.D;
    const cuuint64_t dims[4] = {row, hh, dd, (cuuint64_t)d.N};
    const cuuint64_t st[3] = {row * 2ull, row * 2ull * hh, row * 2ull * hh * dd};
    const cuuint32_t box[4] = {(cuuint32_t)p.raw_row_el, (cuuint32_t)(p.patch_h * p.raw_fh), 1u, 1u};
    const cuuint32_t es[4] = {1u, 1u, 1u, 1u};
    if (enc(&mx, dt, 4, const_cast<void *>(xin), dims, st, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      *detail = "cuTensorMapEncodeTiled failed for the few-channel input";
      return cudaErrorInvalidValue;
    }
  } else if (p.s2_chunks) {   // the caller's [N, D0, H0, W0, C0], H and W traversed with the layer's stride
    const cuuint64_t dims[5] = {(cuuint64_t)d.C0, (cuuint64_t)d.W0, (cuuint64_t)d.H0, (cuuint64_t)d.D0, (cuuint64_t)d.N};
    const cuuint64_t st[4] = {(cuuint64_t)d.C0 * 2ull, (cuuint64_t)d.C0 * 2ull * d.W0, (cuuint64_t)d.C0 * 2ull * d.W0 * d.H0,
                              (cuuint64_t)d.C0 * 2ull * d.W0 * d.H0 * d.D0};
    const cuuint32_t box[5] = {(cuuint32_t)KC, (cuuint32_t)(p.patch_w * d.fW), (cuuint32_t)(p.patch_h * d.fH), 1u, 1u};
    const cuuint32_t es[5] = {1u, (cuuint32_t)d.fW, (cuuint32_t)d.fH, 1u, 1u};
    if (enc(&mx, dt, 5, const_cast<void *>(xin), dims, st, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      *detail = "cuTensorMapEncodeTiled failed for the strided input";
      return cudaErrorInvalidValue;
    }
  } else {
    const cuuint64_t dims[5] = {(cuuint64_t)p.Cp, (cuuint64_t)d.W, (cuuint64_t)d.H, (cuuint64_t)d.D, (cuuint64_t)d.N};
    const cuuint64_t st[4] = {(cuuint64_t)p.Cp * 2ull, (cuuint64_t)p.Cp * 2ull * d.W, (cuuint64_t)p.Cp * 2ull * d.W * d.H,
                              (cuuint64_t)p.Cp * 2ull * d.W * d.H * d.D};
    const cuuint32_t box[5] = {(cuuint32_t)KC, (cuuint32_t)p.patch_w, (cuuint32_t)p.patch_h, 1u, 1u};
    const cuuint32_t es[5] = {1u, 1u, 1u, 1u, 1u};
    if (enc(&mx, dt, 5, const_cast<void *>(xin), dims, st, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      *detail = "cuTensorMapEncodeTiled failed for the input";
      return cudaErrorInvalidValue;
    }
  }
  {
    const cuuint64_t dims[3] = {(cuuint64_t)p.Cp, (cuuint64_t)d.K, (cuuint64_t)p.slabs};
    const cuuint64_t st[2] = {(cuuint64_t)p.Cp * 2ull, (cuuint64_t)p.Cp * 2ull * d.K};
    const cuuint32_t box[3] = {(cuuint32_t)KC, (cuuint32_t)(p.pair ? p.BN / 2 : p.BN), 1u};
    const cuuint32_t es[3] = {1u, 1u, 1u};
    if (enc(&mu, dt, 3, const_cast<void *>(u), dims, st, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      *detail = "cuTensorMapEncodeTiled failed for the transformed filter";
      return cudaErrorInvalidValue;
    }
  }
  int dev = 0, sm_count = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) { *detail = "cudaDeviceGetAttribute(MultiProcessorCount) failed"; return e; }
  const uint32_t fmt = dtype == WINOCONV_F16 ? 0u : 1u;
  const uint32_t m_rows = p.pair ? 2u * BM : (uint32_t)BM;   // a pair's MMA spans the tile blocks of both CTAs
  const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(p.BN >> 3) << 17) | ((m_rows >> 4) << 24);
#define ROWF_DISPATCH(T)                                                                                         \
  do {                                                                                                           \
    if (p.pair) return p.BN == 64 ? launch_rf<T, 64, 1, true>(d, p, mx, mu, y, bias, sm_count, idesc, s, detail) \
                                  : launch_rf<T, 128, 1, true>(d, p, mx, mu, y, bias, sm_count, idesc, s, detail); \
    if (p.MB == 2) return launch_rf<T, 64, 2, false>(d, p, mx, mu, y, bias, sm_count, idesc, s, detail);         \
    return p.BN == 64 ? launch_rf<T, 64, 1, false>(d, p, mx, mu, y, bias, sm_count, idesc, s, detail)            \
                      : launch_rf<T, 128, 1, false>(d, p, mx, mu, y, bias, sm_count, idesc, s, detail);          \
  } while (0)
  if (dtype == WINOCONV_F16) ROWF_DISPATCH(__half);
  ROWF_DISPATCH(__nv_bfloat16);
#undef ROWF_DISPATCH
}


cudaError_t read_and_clear_row_error(cudaStream_t s, unsigned int *code) {
  unsigned int host = 0, zero = 0;
  cudaError_t e = cudaMemcpyFromSymbolAsync(&host, g_row_error, sizeof(host), 0, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaMemcpyToSymbolAsync(g_row_error, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  *code = host;
  return e;
}

}  // namespace wino
