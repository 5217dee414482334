// Tiled tensor-core path for banded masks on sm_100a: TMA-staged K/V tiles, tcgen05 TF32 MMAs with
// TMEM accumulators, online softmax in registers.
//
// One CTA owns 128 * NSUB consecutive query rows of a (strided) row sequence, as NSUB 128-row sub-tiles, and
// walks the key tiles (BN keys each) that intersect the band |u_q - u_k| <= w. Two shapes are launched:
// NSUB = 1 for d <= 64, sized so that two CTAs share an SM and fill each other's gaps (the occupancy API
// reports 1 CTA/SM for any kernel containing tcgen05.alloc; the hardware does co-schedule them), and NSUB = 2
// for d = 128, where one CTA interleaves its two sub-tiles on the tensor pipe. Roles (128 * NSUB + 128 threads):
//   warps 0 .. 4 NSUB-1  softmax groups, one per sub-tile: thread t <-> query row t <-> TMEM lane t
//   next warp            TMA producer (one elected lane) + TMEM allocation
//   next warp            MMA issuer (one elected lane)
//   last two warps       idle (they complete the last warpgroup so registers can be re-balanced with setmaxnreg)
// Per key tile j and sub-tile X (S has two TMEM buffers per sub-tile, used alternately):
//   S_X = Q_X K_j^T      tcgen05.mma kind::tf32, A = Q_X (smem, K-major), B = K_j (smem, K-major), D in TMEM;
//                         issued TWO tiles ahead of the softmax group, so that group never waits for it
//   P_X = exp2(S_X*c - shift) written back over S_X in TMEM by the softmax group (row max / row sum in
//                         registers, no shuffles: one thread owns one row; `shift` is a lazy per-row
//                         reference that moves only when the row maximum outgrows it by 2^8)
//   O_X += P_X V_j       tcgen05.mma kind::tf32, A = P_X (TMEM), B = V_j (smem, MN-major), D stays in TMEM
//                         for the whole CTA; a row whose reference moves rescales its own O row in TMEM
// MMA issue order per key tile j: PV_X(j) for every sub-tile, then S_X(j+2). TMEM per CTA: 2 NSUB S buffers of
// BN columns + NSUB O accumulators of d columns <= 256 NSUB columns.
// Epilogue: O rows leave TMEM through shared memory (the dead Q tile) so that the read-modify-write of
// the caller's O is coalesced.
//
// Strided sequences: the rows a CTA sees are  abs_row = r + u*s  (s = dilation stride, r = residue),
// addressed through tensor maps whose row pitch is s*d*4 bytes; the 1D-dilated mask is exactly a band
// in u on every residue class, Local is s = 1.
//
// Every wait is bounded: on timeout the waiter records a code in *err, raises an abort flag the other
// roles poll, and the CTA falls through to the common exit where TMEM is released.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "spfa_common.cuh"

namespace spfa {
namespace tile {


// Geometry of a CTA with NSUB 128-row sub-tiles: NSUB softmax warpgroups + one warpgroup holding the
// TMA warp, the MMA warp and two idle warps. NSUB = 1 (two CTAs per SM) serves d <= 64, NSUB = 2 (one CTA per
// SM, the sub-tiles interleave on the tensor pipe inside the CTA) serves d = 128.
//
// Register re-balancing. A CTA is launched with Geo::kRegsLaunch registers per thread (what the compiler
// assigns under __launch_bounds__(kThreads, kCtasPerSm)). setmaxnreg.inc BLOCKS until the CTA's pool can
// satisfy it and has no timeout, so the two budgets must fit in the pool the launch allocated -- otherwise
// the softmax groups would wait forever. The host re-checks this against cudaFuncGetAttributes.
template <int NSUB>
struct Geo {
  static constexpr int kThreads = 128 * NSUB + 128;
  static constexpr int kQRows = 128 * NSUB;
  static constexpr int kCtasPerSm = (NSUB == 1) ? 2 : 1;
  static constexpr int kRegsLaunch = (NSUB == 1) ? 128 : 168;
  static constexpr int kRegsSoftmax = (NSUB == 1) ? 208 : 216;
  static constexpr int kRegsAux = (NSUB == 1) ? 48 : 72;
  static constexpr int kSoftmaxWarps = 4 * NSUB;
  static_assert(kRegsSoftmax * 128 * NSUB + kRegsAux * 128 <= kRegsLaunch * kThreads,
                "setmaxnreg budgets exceed the launch pool");
  static_assert(kRegsSoftmax % 8 == 0 && kRegsAux % 8 == 0, "setmaxnreg takes multiples of 8");
};
constexpr uint64_t kWaitNs = 200ull * 1000 * 1000;  // 0.2 s per wait before giving up

struct BandParams {
  int64_t n_keys;     // n_r: rows of this residue's key sequence
  int64_t u_q_first;  // first query u of the shard for this residue
  int64_t n_q;        // number of query rows (u_q_first .. u_q_first + n_q)
  int64_t w;          // band half-width in u
  int64_t s, r;       // stride and residue: abs_row = r + u*s
  int64_t row_begin;  // first absolute row of the shard (Q/m/l/O are indexed by abs_row - row_begin)
  float scale_log2e;  // (1/sqrt(d)) * log2(e)
  // ---- "every key EXCEPT an interval" masks (Global-no-local) ----
  // mode 0: band, a row attends to keys [u-w, u+w] (Local, Local-1D-dilated).
  // mode 1: the keys are the listed global rows, gathered in ascending order (`sorted`, n_keys of them, of
  //         which *n_valid are real); query row i attends to every listed key outside [i-w, i+w]; rows
  //         that are themselves listed are skipped (mode 2 handles them).
  // mode 2: the QUERY rows are the listed global rows (gathered, sorted); row r = sorted[r] attends to
  //         every key of the full sequence outside [sorted[r]-w, sorted[r]+w]. The key range is split
  //         over blockIdx.y (kv_chunk keys per CTA) and each CTA writes a partial softmax state per
  //         row ((d+4) floats: un-normalised O relative to m, then m, l) for a later combine pass.
  // mode 4: band AND listed keys in one pass (fused Local + Global-no-local for the rows that are not listed): a
  //         row attends to the keys [u-w, u+w] of the full sequence (tiles fetched through tmK/tmV) and to every
  //         listed key outside that window (tiles of the gathered listed rows, fetched through tmK2/tmV2);
  //         listed rows are skipped as in mode 1.
  int mode;
  int64_t n_listed;       // modes 1, 4: rows of the gathered listed-key arrays (mode 1: equals n_keys)
  const int32_t* sorted;  // modes 1, 2, 4: ascending global row numbers (invalid entries last, as INT_MAX)
  const int32_t* n_valid; // modes 1, 2: number of real entries in `sorted`
  int64_t kv_chunk;       // mode 2: keys per CTA along blockIdx.y
  float* partials;        // mode 2: [n_keys_of_sorted][n_split][d+4]
  int n_split;            // mode 2: gridDim.y
  // ---- explicit masks (CSR/COO dense tiles; kernel instantiated with EXPL = true) ----
  // The query rows are cut into 128-row blocks (= sub-tiles); block b has x_nt[b] <= kMaxDenseTiles dense key
  // tiles, numbered x_kt[b*kMaxDenseTiles + t] (ascending; tile k covers keys [k*BN, (k+1)*BN)), and for its
  // t-th tile a bit mask of valid (row, key) pairs at x_masks[x_moff[b] + (t*(BN/32) + chunk)*128 + row].
  // ---- overlap with a neighbouring launch of this kernel that touches other rows (dilated masks: one launch
  // per residue class). Bit 0: let the next launch of the stream start as soon as every CTA of this one has
  // started (griddepcontrol.launch_dependents); bit 1: this launch was started that way, so it must not
  // complete before its predecessor has (griddepcontrol.wait before the CTA exits). ----
  int overlap;
  // ---- batches of slices (batch x heads): blockIdx.z selects the slice; Q, K, V come through the third coordinate of
  // the tensor maps, (m, l, O) are offset by these strides (in elements) ----
  int64_t slice_o, slice_ml;
  const int* x_nt;
  const int* x_kt;
  const long long* x_moff;
  const uint32_t* x_masks;
  // explicit masks: the plan's identity block and what the caller expects to find there (every CTA compares them
  // before touching the tables above), and the range of key tiles [x_kt_lo, x_kt_hi) this launch works on (a
  // forward split along the key axis runs one launch per range; the whole mask is [0, INT_MAX); x_kt_lo > x_kt_hi
  // names the cyclic range [x_kt_lo, INT_MAX) + [0, x_kt_hi))
  // ---- bulk store of finished O tiles: set when the launch carries a tensor map of O with Q's geometry (tmO) ----
  int tma_store;
  const PlanHeader* x_hdr;
  PlanHeader x_want;
  int x_kt_lo, x_kt_hi;
};
constexpr int kMaxDenseTiles = 32;  // per 128-row block; a CTA (two blocks) walks at most 64 key tiles

// ---- PTX wrappers ---------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t globaltimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait. Returns false on timeout or when another role raised the abort flag.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err, int code) {
  if (mbar_try(bar, parity)) return true;
  const uint64_t t0 = globaltimer();
  uint32_t spins = 0;
  while (!mbar_try(bar, parity)) {
    if ((++spins & 255u) == 0) {
      if (*abort_flag) return false;
      if (globaltimer() - t0 > kWaitNs) {
        *abort_flag = 1;
        atomicCAS(err, 0, code);
        return false;
      }
    }
  }
  return true;
}

// Tensor maps are rank 3: (element within a row, row, slice). A slice is one [rows, d] matrix of a batch of them
// (batch x heads); unbatched calls have one slice and z = 0.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* tm, int32_t x, int32_t y, int32_t z,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(tm), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t y;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(y) : "f"(x));
  return y;
}

// ---- descriptors ------------------------------------------------------------------------------------
// Shared-memory matrix descriptor, sm_100 format:
//   [0,14) start address >> 4   [16,30) leading byte offset >> 4   [32,46) stride byte offset >> 4
//   [46,48) version = 1         [61,64) layout type
// Layout types used here: 2 = 128-byte swizzle on 16-byte units (K-major operands: Q and K tiles);
// 1 = 128-byte swizzle on 32-byte units, the only layout the hardware accepts for an MN-major 32-bit
// operand (the V tile, whose rows are keys = the contraction dimension of P V).
constexpr uint32_t kLayoutSw128 = 2, kLayoutSw128Base32 = 1;
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3fff);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= 1ull << 46;
  d |= (uint64_t)layout << 61;
  return d;
}

// Instruction descriptor for kind::tf32, fp32 accumulate:
//   [4,6) D format (1 = f32)  [7,10) A format (2 = tf32)  [10,13) B format (2 = tf32)
//   [15] A major (0 = K)  [16] B major (0 = K, 1 = MN)  [17,23) N >> 3  [24,29) M >> 4
__host__ __device__ constexpr uint32_t idesc_tf32(int M, int N, int b_mn_major) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) |
         ((uint32_t)(M >> 4) << 24);
}

// ---- shared-memory plan --------------------------------------------------------------------------------
template <int D, int BN, int NS, int NSUB, int NSV = NS>  // NS: K stages, NSV: V stages
struct Plan {
  static constexpr int kChunks = D / 32;                    // 32-float (128 B) column chunks per row
  static constexpr int kQChunkBytes = 128 * 128;            // 128 rows x 128 B
  static constexpr int kKVChunkBytes = BN * 128;            // BN rows x 128 B
  static constexpr int kQBytes = NSUB * kChunks * kQChunkBytes;  // all sub-tiles
  static constexpr int kKVStageBytes = kChunks * kKVChunkBytes;
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = kOffQ + kQBytes;
  static constexpr int kOffV = kOffK + NS * kKVStageBytes;
  static constexpr int kOffBar = kOffV + NSV * kKVStageBytes;
  // barriers: q_full, k_full[NS], k_empty[NS], v_full[NSV], v_empty[NSV], s_ready[2 NSUB], p_ready[2 NSUB], o_ready[2 NSUB] (one per S buffer / tile parity)
  static constexpr int kNumBars = 1 + 2 * NS + 2 * NSV + 6 * NSUB;
  static constexpr int kOffMisc = kOffBar + kNumBars * 8;   // tmem base (4 B), abort flag (4 B)
  // explicit masks: merged key-tile list of the CTA: kt[64] (int), act[NSUB] (u64, bit j = sub-tile uses tile j;
  // tile j is then the popcount(act & (2^j - 1))-th tile of the sub-tile's own list), nT (int)
  static constexpr int kOffX = (kOffMisc + 16 + 15) / 16 * 16;
  // pos[NSUB][64] (u8): position of the CTA's tile j in sub-tile x's own list (where its bit masks are stored)
  static constexpr int kXKt = 0, kXAct = 256, kXNt = 256 + 8 * NSUB, kXPos = kXNt + 4;
  static constexpr int kBytesCore = kOffX + (kXPos + 64 * NSUB + 15) / 16 * 16;
  // mode 1 (rows x listed keys): a copy of the sorted list (<= 1024 entries) for the per-row interval searches, where
  // the CTA's shared memory has room for it (every shape but the two-sub-tile d = 128 one, which never runs mode 1
  // from the library's dispatch and would search in global memory)
  static constexpr int kSortedBytes = 4096;
  static constexpr bool kStageSorted = kBytesCore + kSortedBytes + 1024 <= 227 * 1024;
  static constexpr int kOffSorted = kBytesCore;
  static constexpr int kBytes = kBytesCore + (kStageSorted ? kSortedBytes : 0);
  static constexpr int kDynSmem = kBytes + 1024;            // slack for 1024-B alignment of the base
  static_assert(kDynSmem <= 227 * 1024, "beyond the shared memory one CTA can opt into");
  // TMEM columns: two S buffers per sub-tile (BN each, at BN (2x + b)), then O_x (D each, at 2 BN NSUB + D x)
  static constexpr int kTmemCols = 256 * NSUB;
  static constexpr int kColS = 0, kColO = 2 * BN * NSUB;
  static_assert(kColO + NSUB * D <= kTmemCols, "S buffers and O accumulators exceed the TMEM allocation");
};

template <int D, int BN, int NS, int NSUB, bool EXPL = false, int NSV = NS>
__global__ void __launch_bounds__(Geo<NSUB>::kThreads, Geo<NSUB>::kCtasPerSm)
band_forward_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmK2,
                    const __grid_constant__ CUtensorMap tmV2, const __grid_constant__ CUtensorMap tmO,
                    float* __restrict__ m_base, float* __restrict__ l_base, float* __restrict__ O_base,
                    const BandParams prm, int* __restrict__ err) {
  const int32_t zs = (int32_t)blockIdx.z;  // slice of a batched call
  float* __restrict__ m_out = m_base + (size_t)zs * prm.slice_ml;
  float* __restrict__ l_out = l_base + (size_t)zs * prm.slice_ml;
  float* __restrict__ O_out = O_base + (size_t)zs * prm.slice_o;
  using P = Plan<D, BN, NS, NSUB, NSV>;
  using G = Geo<NSUB>;
  constexpr int kQRows = G::kQRows;
  constexpr int W_TMA = G::kSoftmaxWarps, W_MMA = G::kSoftmaxWarps + 1;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + P::kOffBar;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  const int B_QFULL = 0, B_KFULL = 1, B_KEMPTY = 1 + NS, B_VFULL = 1 + 2 * NS, B_VEMPTY = 1 + 2 * NS + NSV,
            B_SREADY = 1 + 2 * NS + 2 * NSV, B_PREADY = B_SREADY + 2 * NSUB, B_OREADY = B_SREADY + 4 * NSUB;
  volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(smem + P::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + P::kOffMisc + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Explicit masks: the block's tile counts and mask offset are asked for together with the plan's identity block, one
  // round trip instead of three. The host has checked that the plan region is at least as large as the layout of the
  // shape the caller passed, so these reads stay inside it even when the identity block turns out to differ.
  int nt_early[NSUB];
  long long moff_early = 0;
#pragma unroll
  for (int x = 0; x < NSUB; ++x) nt_early[x] = 0;
  if (EXPL) {
    const int64_t n_blocks_e = (prm.n_q + 127) / 128;
#pragma unroll
    for (int x = 0; x < NSUB; ++x) {
      const int64_t b = (int64_t)blockIdx.x * NSUB + x;
      if (b < n_blocks_e) nt_early[x] = prm.x_nt[b];
    }
    const int64_t bq = (int64_t)blockIdx.x * NSUB + (((warp >> 2) < NSUB) ? (warp >> 2) : (NSUB - 1));
    if (bq < n_blocks_e) moff_early = prm.x_moff[bq];
  }
  if (EXPL) {  // uniform over the CTA: a plan of another shape is not walked at all
    if (!plan_header_matches(prm.x_hdr, prm.x_want)) {
      if (threadIdx.x == 0) atomicCAS(err, 0, kPlanMismatchCode);
      if ((prm.overlap & 2) && threadIdx.x == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
      return;
    }
  }

  // ---- tile geometry (uniform across the CTA) ----
  const int64_t uq0 = prm.u_q_first + (int64_t)blockIdx.x * kQRows;  // first query u of this CTA
  const int64_t uq_end = prm.u_q_first + prm.n_q;                    // one past the last valid query u
  const int64_t rows_here = (uq_end - uq0 < kQRows) ? (uq_end - uq0) : kQRows;
  int64_t kv_lo, kv_hi;
  int64_t uq_end_eff = uq_end;  // mode 2: only the real entries of the sorted list are query rows
  if (EXPL) {
    kv_lo = 0;
    kv_hi = prm.n_keys;
  } else if (prm.mode == 0 || prm.mode == 4) {
    kv_lo = (uq0 - prm.w > 0) ? (uq0 - prm.w) : 0;
    kv_hi = uq0 + rows_here - 1 + prm.w + 1;
    if (kv_hi > prm.n_keys) kv_hi = prm.n_keys;
  } else if (prm.mode == 1) {
    kv_lo = 0;
    kv_hi = *prm.n_valid;  // real listed keys
    if (kv_hi > prm.n_keys) kv_hi = prm.n_keys;
  } else {
    kv_lo = (int64_t)blockIdx.y * prm.kv_chunk;
    kv_hi = kv_lo + prm.kv_chunk;
    if (kv_hi > prm.n_keys) kv_hi = prm.n_keys;
    if (uq_end_eff > *prm.n_valid) uq_end_eff = *prm.n_valid;
  }
  if (kv_hi < kv_lo) kv_hi = kv_lo;
  int nT = (int)((kv_hi - kv_lo + BN - 1) / BN);
  // mode 4: the band's tiles are followed by the tiles of the listed keys (every sub-tile with rows uses all of them)
  const int nTb = nT;
  int nv4 = 0;  // mode 4: real listed keys
  if (!EXPL && prm.mode == 4) {
    nv4 = *prm.n_valid;
    if (nv4 > prm.n_listed) nv4 = (int)prm.n_listed;
    nT += (nv4 + BN - 1) / BN;
  }
  // Key tiles of each sub-tile: a contiguous range [j0, j1) of the CTA's tiles (implicit masks), or the set
  // bits of act[x] over the CTA's merged tile list (explicit masks, read from shared memory after set-up).
  int j0[NSUB], j1[NSUB], jl[NSUB];  // jl: first listed-key tile of the sub-tile (mode 4), else "never"
  uint64_t act[NSUB];
  const int* s_kt = reinterpret_cast<const int*>(smem + P::kOffX + P::kXKt);
#pragma unroll
  for (int x = 0; x < NSUB; ++x) {
    act[x] = 0;
    jl[x] = 0x7fffffff;
    const int64_t ux0 = uq0 + 128 * x;
    int64_t ux_last = ux0 + 127;
    if (ux_last > uq_end_eff - 1) ux_last = uq_end_eff - 1;
    if (ux0 >= uq_end_eff) {
      j0[x] = 0;
      j1[x] = 0;
    } else if (prm.mode != 0 && prm.mode != 4) {
      j0[x] = 0;
      j1[x] = nT;
    } else {
      const int64_t lo = (ux0 - prm.w > 0) ? (ux0 - prm.w) : 0;
      int64_t hi = ux_last + prm.w + 1;
      if (hi > prm.n_keys) hi = prm.n_keys;
      j0[x] = (int)((lo - kv_lo) / BN);
      j1[x] = (int)((hi - kv_lo + BN - 1) / BN);
      if (prm.mode == 4) jl[x] = nTb;
    }
  }

  // ---- setup ----
  if ((prm.overlap & 1) && threadIdx.x == 96) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 64) {  // descriptor fetches off the first loads' critical path
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmQ)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmK)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmV)) : "memory");
  }
  if (threadIdx.x == 0) {
    mbar_init(bar(B_QFULL), 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(bar(B_KFULL + s), 1);
      mbar_init(bar(B_KEMPTY + s), 1);
    }
    for (int s = 0; s < NSV; ++s) {
      mbar_init(bar(B_VFULL + s), 1);
      mbar_init(bar(B_VEMPTY + s), 1);
    }
    for (int x = 0; x < 2 * NSUB; ++x) {
      mbar_init(bar(B_SREADY + x), 1);
      mbar_init(bar(B_PREADY + x), 128);
      mbar_init(bar(B_OREADY + x), 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (EXPL && warp == 1) {
    // Merge the ascending dense-tile lists of the CTA's sub-tiles into one ascending list of key tiles. The lists are
    // fetched by the whole warp first (one entry per lane, kMaxDenseTiles = 32) into the Q region, which stays free
    // until the barrier below: a single thread walking them in global memory paid a round trip per entry.
    static_assert(kMaxDenseTiles <= 32, "one list entry per lane");
    int* s_list = reinterpret_cast<int*>(smem + P::kOffQ);
    {
      const int64_t n_blocks_w = (prm.n_q + 127) / 128;
#pragma unroll
      for (int x = 0; x < NSUB; ++x) {
        const int64_t b = (int64_t)blockIdx.x * NSUB + x;
        int nx_w = (b < n_blocks_w) ? nt_early[x] : 0;
        if (nx_w > kMaxDenseTiles) nx_w = kMaxDenseTiles;
        if (nx_w < 0) nx_w = 0;
        s_list[x * 32 + lane] = (lane < nx_w) ? __ldg(prm.x_kt + b * kMaxDenseTiles + lane) : 0x7fffffff;
      }
    }
    __syncwarp();
  }
  if (EXPL && threadIdx.x == 32) {
    int* kt = reinterpret_cast<int*>(smem + P::kOffX + P::kXKt);
    uint64_t* s_act = reinterpret_cast<uint64_t*>(smem + P::kOffX + P::kXAct);
    const int64_t n_blocks = (prm.n_q + 127) / 128;
    int n[NSUB], pos[NSUB];
    const int* list[NSUB];
    const int* s_list_ro = reinterpret_cast<const int*>(smem + P::kOffQ);
    uint64_t a[NSUB];
    uint8_t* s_pos = smem + P::kOffX + P::kXPos;
    // key tiles this launch works on: [lo, hi), or the cyclic range [lo, inf) + [0, hi) when lo > hi
    const int lo = prm.x_kt_lo, hi = prm.x_kt_hi;
    auto wanted = [&](int k) { return (lo <= hi) ? (k >= lo && k < hi) : (k >= lo || k < hi); };
#pragma unroll
    for (int x = 0; x < NSUB; ++x) {
      const int64_t b = (int64_t)blockIdx.x * NSUB + x;
      n[x] = (b < n_blocks) ? nt_early[x] : 0;
      if (n[x] > kMaxDenseTiles) n[x] = kMaxDenseTiles;
      if (n[x] < 0) n[x] = 0;
      list[x] = s_list_ro + x * 32;
      pos[x] = 0;
      a[x] = 0;
      while (pos[x] < n[x] && !wanted(list[x][pos[x]])) ++pos[x];
    }
    int nt = 0;
    while (nt < 64) {
      int best = 0x7fffffff;
#pragma unroll
      for (int x = 0; x < NSUB; ++x)
        if (pos[x] < n[x]) {
          const int k = list[x][pos[x]];
          best = (k < best) ? k : best;
        }
      if (best == 0x7fffffff) break;
      kt[nt] = best;
#pragma unroll
      for (int x = 0; x < NSUB; ++x)
        if (pos[x] < n[x] && list[x][pos[x]] == best) {
          a[x] |= 1ull << nt;
          s_pos[x * 64 + nt] = (uint8_t)pos[x];
          ++pos[x];
          while (pos[x] < n[x] && !wanted(list[x][pos[x]])) ++pos[x];
        }
      ++nt;
    }
#pragma unroll
    for (int x = 0; x < NSUB; ++x) s_act[x] = a[x];
    *reinterpret_cast<int*>(smem + P::kOffX + P::kXNt) = nt;
  }
  if (!EXPL && P::kStageSorted && (prm.mode == 1 || prm.mode == 4)) {
    int32_t* s_sorted = reinterpret_cast<int32_t*>(smem + P::kOffSorted);
    const int cap = (prm.n_listed < P::kSortedBytes / 4) ? (int)prm.n_listed : P::kSortedBytes / 4;
    for (int i = threadIdx.x; i < cap; i += G::kThreads) s_sorted[i] = __ldg(prm.sorted + i);
  }
  if (warp == W_TMA) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sbase + P::kOffMisc),
                 "r"(P::kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_base_slot;
  if (EXPL) {
    nT = *reinterpret_cast<const int*>(smem + P::kOffX + P::kXNt);
#pragma unroll
    for (int x = 0; x < NSUB; ++x) act[x] = reinterpret_cast<const uint64_t*>(smem + P::kOffX + P::kXAct)[x];
  }
  // helpers over both representations of "sub-tile x uses key tile j"
  auto active = [&](int x, int j) -> bool {
    return EXPL ? (((act[x] >> j) & 1ull) != 0) : ((j >= j0[x] && j < j1[x]) || j >= jl[x]);
  };
  auto it_of = [&](int x, int j) -> int {  // how many of x's tiles come before tile j
    return EXPL ? __popcll(act[x] & ((1ull << j) - 1ull)) : ((j < nTb) ? (j - j0[x]) : (j1[x] - j0[x] + j - nTb));
  };
  auto tile_key0 = [&](int j) -> int32_t {  // first key row of the CTA's tile j (listed-key tiles: row of the gathered array)
    return EXPL ? (int32_t)(s_kt[j] * BN)
                : ((j < nTb) ? (int32_t)(kv_lo + (int64_t)j * BN) : (int32_t)((j - nTb) * BN));
  };

  if (warp >= W_TMA) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(G::kRegsAux));
  if (warp == W_TMA) {
    // =============================== TMA producer ===============================
    if (lane == 0 && nT > 0) {  // nothing is fetched for a CTA without key tiles (no listed key at all)
      // Q: both sub-tiles, coordinates relative to the first query u of the shard (rows past the end read zeros)
      mbar_expect_tx(bar(B_QFULL), P::kQBytes);
      const int32_t yq = (int32_t)(uq0 - prm.u_q_first);
#pragma unroll
      for (int x = 0; x < NSUB; ++x)
#pragma unroll
        for (int c = 0; c < P::kChunks; ++c)
          tma_load_3d(sbase + P::kOffQ + (x * P::kChunks + c) * P::kQChunkBytes, &tmQ, c * 32, yq + 128 * x, zs,
                      bar(B_QFULL));
      // K runs NS tiles ahead of V (the S MMAs are issued ahead of the softmax, the PV MMAs behind it), so the
      // order is K(0..NS-1), then V(j), K(j+NS) for every tile j: a wait for a V stage never holds back a K tile
      // that the MMA thread needs first.
      bool ok = true;
      auto load_k = [&](int j) -> bool {
        const int st = j % NS;
        if (!mbar_wait(bar(B_KEMPTY + st), (uint32_t)((j / NS) & 1) ^ 1u, abort_flag, err, 101)) return false;
        mbar_expect_tx(bar(B_KFULL + st), P::kKVStageBytes);
        const int32_t yk = tile_key0(j);
#pragma unroll
        for (int c = 0; c < P::kChunks; ++c)
          tma_load_3d(sbase + P::kOffK + st * P::kKVStageBytes + c * P::kKVChunkBytes, (j < nTb) ? &tmK : &tmK2, c * 32, yk,
                      zs, bar(B_KFULL + st));
        return true;
      };
      for (int j = 0; j < NS && j < nT && ok; ++j) ok = load_k(j);
      for (int j = 0; j < nT && ok; ++j) {
        const int st = j % NSV;
        ok = mbar_wait(bar(B_VEMPTY + st), (uint32_t)((j / NSV) & 1) ^ 1u, abort_flag, err, 102);
        if (!ok) break;
        mbar_expect_tx(bar(B_VFULL + st), P::kKVStageBytes);
        const int32_t yk = tile_key0(j);
#pragma unroll
        for (int c = 0; c < P::kChunks; ++c)
          tma_load_3d(sbase + P::kOffV + st * P::kKVStageBytes + c * P::kKVChunkBytes, (j < nTb) ? &tmV : &tmV2, c * 32, yk,
                      zs, bar(B_VFULL + st));
        if (j + NS < nT) ok = load_k(j + NS);
      }
    }
  } else if (warp == W_MMA) {
    // =============================== MMA issuer ===============================
    if (lane == 0) {
      constexpr uint32_t kIdescS = idesc_tf32(128, BN, 0);
      constexpr uint32_t kIdescO = idesc_tf32(128, D, 1);
      bool ok = (nT > 0) && mbar_wait(bar(B_QFULL), 0, abort_flag, err, 201);
      // Descriptors are built once per operand tile; each MMA only adds a compile-time offset to the
      // 14-bit start-address field (shared memory is < 256 KB, so the field cannot carry out).
      // S of a sub-tile's it-th key tile goes to its S buffer it & 1; it is issued two tiles ahead of the
      // softmax group so that group never waits for the tensor pipe.
      auto issue_S = [&](int x, int j) {
        const int st = j % NS;
        const int sb = x * 2 + (it_of(x, j) & 1);
        const uint64_t qd = smem_desc(sbase + P::kOffQ + x * P::kChunks * P::kQChunkBytes, 16, 1024, kLayoutSw128);
        const uint64_t kd = smem_desc(sbase + P::kOffK + st * P::kKVStageBytes, 16, 1024, kLayoutSw128);
        const uint32_t d_t = tmem + P::kColS + BN * sb;
#pragma unroll
        for (int c = 0; c < P::kChunks; ++c)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_ss(d_t, qd + (uint64_t)((c * P::kQChunkBytes + kk * 32) >> 4),
                   kd + (uint64_t)((c * P::kKVChunkBytes + kk * 32) >> 4), kIdescS, (c | kk) ? 1u : 0u);
        tc_commit(bar(B_SREADY + sb));
      };
      auto issue_PV = [&](int x, int j) {
        const int st = j % NSV;
        const int it = it_of(x, j);
        const int sb = x * 2 + (it & 1);
        // 8 keys per MMA = two 4-row swizzle groups (stride 512 B); 32-dim blocks are kKVChunkBytes apart
        const uint64_t vd = smem_desc(sbase + P::kOffV + st * P::kKVStageBytes, P::kKVChunkBytes, 512, kLayoutSw128Base32);
        const uint32_t a_t = tmem + P::kColS + BN * sb;
        const uint32_t d_t = tmem + P::kColO + D * x;
        const uint32_t first = (it > 0) ? 1u : 0u;  // O accumulates in TMEM across the key tiles of a sub-tile
#pragma unroll
        for (int kk = 0; kk < BN / 8; ++kk)
          mma_ts(d_t, a_t + kk * 8, vd + (uint64_t)((kk * 1024) >> 4), kIdescO, kk > 0 ? 1u : first);
        tc_commit(bar(B_OREADY + sb));  // tiles alternate between two barriers, like the S buffers
      };
      auto last_active = [&](int x, int j) {  // is x the last sub-tile (in issue order A, B) using tile j?
        return x == NSUB - 1 || !active(NSUB - 1, j);
      };
      // S of key tile jj for every sub-tile that uses it, then release the K stage
      auto issue_S_tile = [&](int jj) -> bool {
        if (jj >= nT) return true;
        if (!mbar_wait(bar(B_KFULL + jj % NS), (uint32_t)((jj / NS) & 1), abort_flag, err, 202)) return false;
        tc_fence_after();
        for (int x = 0; x < NSUB; ++x)
          if (active(x, jj)) {
            issue_S(x, jj);
            if (last_active(x, jj)) tc_commit(bar(B_KEMPTY + jj % NS));
          }
        return true;
      };
      // prologue: S of key tiles 0 and 1
      ok = ok && issue_S_tile(0);
      ok = ok && issue_S_tile(1);
      for (int j = 0; j < nT && ok; ++j) {
        const int st = j % NSV;
        const uint32_t ph = (uint32_t)((j / NSV) & 1);
        bool have_v = false;
        for (int x = 0; x < NSUB && ok; ++x) {
          if (!active(x, j)) continue;
          const int it = it_of(x, j);
          ok = mbar_wait(bar(B_PREADY + x * 2 + (it & 1)), (uint32_t)((it >> 1) & 1), abort_flag, err, 203);
          if (!ok) break;
          if (!have_v) {
            ok = mbar_wait(bar(B_VFULL + st), ph, abort_flag, err, 204);
            if (!ok) break;
            have_v = true;
          }
          tc_fence_after();
          issue_PV(x, j);
          if (last_active(x, j)) tc_commit(bar(B_VEMPTY + st));
        }
        // the S buffers of tile j are free again once its PVs are queued (the pipe runs them in order)
        ok = ok && issue_S_tile(j + 2);
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(G::kRegsSoftmax));
    // =============================== softmax groups ===============================
    // One thread owns one query row. Per key tile the row of S is read from TMEM ONCE (all chunk loads
    // issued back to back), exponentiated against a per-row reference `shift`, and written back as P.
    // O accumulates in TMEM across tiles (the PV MMAs add into it), so nothing is read back per tile.
    // `shift` is lazy: it only moves when the row maximum exceeds it by more than kShiftSlack (log2
    // units), in which case this thread rescales its own O row and row sum. The true running maximum is
    // tracked separately for the (m, l) state the caller gets back.
    constexpr int NC = BN / 32;              // 32-column chunks per key tile
    constexpr float kShiftSlack = 8.0f;      // P values stay below 2^8 relative to the reference
    const int x = warp >> 2;                 // sub-tile
    const int row = threadIdx.x & 127;       // row within the sub-tile == TMEM lane
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS0 = tmem + lane_base + P::kColS + 2 * BN * x;
    const uint32_t tO = tmem + lane_base + P::kColO + D * x;
    const int64_t uq = uq0 + 128 * x + row;
    const bool row_valid = uq < uq_end_eff;
    // Per-row key interval [lo_q, hi_q] as 32-bit offsets from the CTA's first key tile: the keys a row
    // attends to (mode 0) or the keys it must skip (modes 1, 2). Both ends grow with the row, so the first
    // and last row of a warp (lo_a/hi_a, lo_b/hi_b) bound every row of the warp: that makes the chunk
    // classes below warp-uniform.
    int lo_q = 0, hi_q = -1;
    int lo2_q = 0, hi2_q = -1;  // mode 4: the listed keys (positions in the sorted list) this row must skip
    bool listed = false;  // modes 1, 4: this query row is itself a global row (handled by the mode-2 launch)
    if (EXPL) {
      lo_q = hi_q = 0;  // validity comes from the plan's bit masks
    } else if (prm.mode == 0 || prm.mode == 4) {
      const int64_t n1 = prm.n_keys - 1;
      lo_q = (int)(((uq - prm.w > 0) ? (uq - prm.w) : 0) - kv_lo);
      hi_q = (int)(((uq + prm.w < n1) ? (uq + prm.w) : n1) - kv_lo);
    }
    if (!EXPL && (prm.mode == 1 || prm.mode == 4)) {
      const int nv = (prm.mode == 1) ? (int)kv_hi : nv4;
      const int64_t ic = (uq < uq_end - 1) ? uq : (uq_end - 1);  // clamp keeps the bounds monotone past the end
      const int32_t* s_sorted = reinterpret_cast<const int32_t*>(smem + P::kOffSorted);
      const bool staged = P::kStageSorted && prm.n_listed <= P::kSortedBytes / 4;
      auto entry = [&](int t) -> int64_t { return staged ? (int64_t)s_sorted[t] : (int64_t)__ldg(prm.sorted + t); };
      auto lower_bound = [&](int64_t v) {  // first t with sorted[t] >= v
        int a = 0, b = nv;
        while (a < b) {
          const int mid = (a + b) >> 1;
          if (entry(mid) < v) a = mid + 1; else b = mid;
        }
        return a;
      };
      const int sk_lo = lower_bound(ic - prm.w), sk_hi = lower_bound(ic + prm.w + 1) - 1;
      if (prm.mode == 1) {
        lo_q = sk_lo;
        hi_q = sk_hi;
      } else {
        lo2_q = sk_lo;
        hi2_q = sk_hi;
      }
      const int t = lower_bound(ic);
      listed = (t < nv) && (entry(t) == ic);
    } else if (!EXPL && prm.mode == 2) {
      const int nv = *prm.n_valid;
      const int64_t rc = (uq < nv - 1) ? uq : (int64_t)(nv - 1);
      const int64_t g = (nv > 0) ? (int64_t)__ldg(prm.sorted + (rc > 0 ? rc : 0)) : 0;
      const int64_t a = g - prm.w - kv_lo, b = g + prm.w - kv_lo;
      lo_q = (int)((a < -(1 << 30)) ? -(1 << 30) : ((a > (1 << 30)) ? (1 << 30) : a));
      hi_q = (int)((b < -(1 << 30)) ? -(1 << 30) : ((b > (1 << 30)) ? (1 << 30) : b));
    }
    const int lo_a = __shfl_sync(kFullMask, lo_q, 0), lo_b = __shfl_sync(kFullMask, lo_q, 31);
    const int hi_a = __shfl_sync(kFullMask, hi_q, 0), hi_b = __shfl_sync(kFullMask, hi_q, 31);
    const int lo2_a = __shfl_sync(kFullMask, lo2_q, 0), lo2_b = __shfl_sync(kFullMask, lo2_q, 31);
    const int hi2_a = __shfl_sync(kFullMask, hi2_q, 0), hi2_b = __shfl_sync(kFullMask, hi2_q, 31);
    const int n_cols = (int)(kv_hi - kv_lo);  // real keys of this CTA's range
    // The caller's state row is needed only in the epilogue. Its (m, l) are read now, off the end of the CTA, and
    // decide what the epilogue must fetch: a row whose l is 0 carries no information -- its old O row is multiplied by
    // 0 -- so the D*4 bytes are neither prefetched nor read (a third of the traffic of a launch whose rows have few
    // keys). The one exception the reference's arithmetic has, 0 * NaN = NaN for a row that an earlier use_nan call
    // filled, is kept: the row's first element is looked at, and a row that does not start with a finite value is
    // read in full like a row with l > 0. Other rows of the launch are never touched by this CTA, and launches that
    // overlap (prm.overlap) write disjoint rows, so reading the state this early sees its final value. A CTA with
    // many key tiles looks at the three values right away (its softmax warps wait for the first S tile anyway); one with
    // a handful of tiles only issues the loads here and looks at them after its first tile, so that their latency does
    // not hold that tile up.
    const bool has_state = row_valid && prm.mode != 2 && !listed;
    float m_in0 = neg_inf(), l_in0 = 0.f, o_first = 0.f;
    auto prefetch_old_row = [&]() {
      if (has_state && !((l_in0 == 0.f) && (fabsf(o_first) <= 3.402823466e38f))) {
        const char* orow = reinterpret_cast<const char*>(O_out + (size_t)(prm.r + uq * prm.s - prm.row_begin) * D);
#pragma unroll
        for (int b = 0; b < D * 4; b += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(orow + b));
      }
    };
    if (has_state) {
      const int64_t rl0 = prm.r + uq * prm.s - prm.row_begin;
      m_in0 = m_out[rl0];
      l_in0 = l_out[rl0];
      o_first = O_out[(size_t)rl0 * D];
    }
    float m_true = neg_inf();   // running maximum of the scaled scores (log2 units)
    float shift = neg_inf();    // reference the exponentials and O are currently expressed against
    float l_run = 0.f;          // row sum relative to `shift`
    bool ok = true;
    uint32_t sr[NC][32];
    const int n_band = j1[x] - j0[x];
    const int nx = EXPL ? __popcll(act[x]) : (n_band + ((jl[x] != 0x7fffffff) ? (nT - nTb) : 0));
    const float sc = prm.scale_log2e;
    const bool early_look = nx > 6;  // uniform over the softmax group
    if (early_look) prefetch_old_row();
    uint64_t rem = act[x];  // explicit masks: tiles of this sub-tile not yet visited
    const uint32_t* xm = nullptr;
    if (EXPL && nx > 0) xm = prm.x_masks + moff_early + row;  // (warp >> 2 == x for the softmax warps)
    const uint8_t* x_pos = smem + P::kOffX + P::kXPos + x * 64;  // explicit masks: tile j -> position in the block's list
    // Explicit masks: the row's mask words of a tile come from global memory and decide the tile's chunk classes, so a
    // load issued when the tile starts would put a DRAM round trip in front of every tile. They are loaded one tile
    // ahead instead: the first tile's words travel while Q and the first S are on their way.
    uint32_t vm_next[NC];
#pragma unroll
    for (int c = 0; c < NC; ++c) vm_next[c] = 0u;
    auto load_masks = [&](int jj) {
#pragma unroll
      for (int c = 0; c < NC; ++c) vm_next[c] = __ldg(xm + (size_t)(x_pos[jj] * NC + c) * 128);
    };
    if (EXPL && nx > 0) load_masks(__ffsll((long long)rem) - 1);
    for (int it = 0; it < nx && ok; ++it) {
      int j;
      uint32_t vm_cur[NC];
#pragma unroll
      for (int c = 0; c < NC; ++c) vm_cur[c] = vm_next[c];
      if (EXPL) {
        j = __ffsll((long long)rem) - 1;
        rem &= rem - 1;
        if (rem) load_masks(__ffsll((long long)rem) - 1);
      } else {
        j = (it < n_band) ? (j0[x] + it) : (nTb + it - n_band);
      }
      // mode 4 switches per tile between "keys inside the band" (band tiles) and "listed keys outside the window"
      const bool lst = !EXPL && prm.mode == 4 && j >= nTb;
      const int tmode = lst ? 1 : ((prm.mode == 4) ? 0 : prm.mode);
      const int k0 = (lst ? (j - nTb) : j) * BN;
      // Interval of this tile's columns: this row [c_lo, c_hi]; common to every row of the warp [w_lo, w_hi];
      // touched by some row of the warp [v_lo, v_hi]  (lo and hi grow with the row)
      const int c_lo = (lst ? lo2_q : lo_q) - k0, c_hi = (lst ? hi2_q : hi_q) - k0;
      const int w_lo = (lst ? lo2_b : lo_b) - k0, w_hi = (lst ? hi2_a : hi_a) - k0;
      const int v_lo = (lst ? lo2_a : lo_a) - k0, v_hi = (lst ? hi2_b : hi_b) - k0;
      const int nvc = (lst ? nv4 : n_cols) - k0;  // columns of this tile that are real keys
      // Chunk classes (warp-uniform): 2 = every (row, column) valid, 0 = none valid, 1 = mixed.
      // Mixed chunks use a per-row bit mask of valid columns.
      int cls[NC];
      uint32_t vmask[NC];
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const int cb = c * 32;
        const int a = c_lo - cb, b = c_hi - cb;  // this row's interval within the chunk, clipped to [0, 31]
        const uint32_t m_lo = (a <= 0) ? 0xffffffffu : (a >= 32 ? 0u : (0xffffffffu << a));
        const uint32_t m_hi = (b >= 31) ? 0xffffffffu : (b < 0 ? 0u : (0xffffffffu >> (31 - b)));
        const uint32_t m_in = m_lo & m_hi;
        if (EXPL) {  // valid = the pair's bit in the plan (masks are stored by the tile's position in the block's own list)
          const uint32_t vm = vm_cur[c];
          vmask[c] = vm;
          cls[c] = __all_sync(kFullMask, vm == 0xffffffffu) ? 2 : (__all_sync(kFullMask, vm == 0u) ? 0 : 1);
        } else if (tmode == 0) {  // valid = inside the interval
          cls[c] = (cb >= w_lo && cb + 31 <= w_hi) ? 2 : ((cb + 31 < v_lo || cb > v_hi) ? 0 : 1);
          vmask[c] = m_in;
        } else {              // valid = a real key outside the interval
          const int r = nvc - cb;
          const uint32_t m_rng = (r >= 32) ? 0xffffffffu : (r <= 0 ? 0u : ((1u << r) - 1u));
          const bool all_valid = (r >= 32) && (cb + 31 < v_lo || cb > v_hi);
          const bool none_valid = (r <= 0) || (cb >= w_lo && cb + 31 <= w_hi);
          cls[c] = all_valid ? 2 : (none_valid ? 0 : 1);
          vmask[c] = m_rng & ~m_in;
        }
      }
      const int sb = x * 2 + (it & 1);                  // S buffer of this tile
      const uint32_t tS = tS0 + BN * (it & 1);
      ok = __all_sync(kFullMask, mbar_wait(bar(B_SREADY + sb), (uint32_t)((it >> 1) & 1), abort_flag, err, 301));
      if (!ok) break;
      tc_fence_after();
      // ---- the whole S row, one TMEM latency ----
#pragma unroll
      for (int c = 0; c < NC; ++c)
        if (cls[c] != 0) tmem_ld32(tS + c * 32, sr[c]);
      tc_wait_ld();
      // ---- row maximum over the valid columns ----
      float mx[4] = {neg_inf(), neg_inf(), neg_inf(), neg_inf()};
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        if (cls[c] == 2) {
#pragma unroll
          for (int e = 0; e < 32; ++e) mx[e & 3] = fmaxf(mx[e & 3], __uint_as_float(sr[c][e]));
        } else if (cls[c] == 1) {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            mx[e & 3] = fmaxf(mx[e & 3], ((vmask[c] >> e) & 1u) ? __uint_as_float(sr[c][e]) : neg_inf());
        }
      }
      const float t_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * sc;  // sc > 0
      m_true = fmaxf(m_true, t_max);
      // ---- move the reference if this row outgrew it (always on the row's first valid tile) ----
      const bool move = t_max > shift + kShiftSlack;  // shift = -inf: true as soon as the row has a valid column
      if (__any_sync(kFullMask, move)) {
        const float new_shift = move ? t_max : shift;
        const float f = move ? ((shift == neg_inf()) ? 0.f : fast_exp2(shift - new_shift)) : 1.0f;
        l_run *= f;
        if (it > 0) {
          // O of this row must be final up to the previous tile before it is rescaled: wait for that PV
          // (the PV of this tile cannot start before our P is ready). PV completions alternate between
          // two barriers per sub-tile, so this parity wait is unambiguous: the barrier of tile it-1 can be
          // neither two phases behind (S of this tile was queued after the PV of tile it-3 on it) nor
          // ahead (tile it+1 needs a P this group has not produced).
          ok = __all_sync(kFullMask, mbar_wait(bar(B_OREADY + x * 2 + ((it - 1) & 1)), (uint32_t)(((it - 1) >> 1) & 1),
                                               abort_flag, err, 302));
          if (!ok) break;
          tc_fence_after();
          uint32_t ob[8];  // small pieces: the S row (sr) stays live in registers across this
#pragma unroll 1
          for (int c = 0; c < D / 8; ++c) {
            tmem_ld8(tO + c * 8, ob);
            tc_wait_ld();
#pragma unroll
            for (int e = 0; e < 8; ++e) ob[e] = __float_as_uint(__uint_as_float(ob[e]) * f);
            tmem_st8(tO + c * 8, ob);
          }
        }
        shift = new_shift;
      }
      const float neg_shift = (shift == neg_inf()) ? 0.f : -shift;
      // ---- P = exp2(S*sc - shift) truncated to tf32 (the bits the MMA reads); the row sum adds the
      //      truncated values so that P / l stays exactly normalised; P goes back over S ----
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        if (cls[c] == 2) {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const uint32_t pb = __float_as_uint(fast_exp2(fmaf(__uint_as_float(sr[c][e]), sc, neg_shift))) & 0xffffe000u;
            ls[e & 3] += __uint_as_float(pb);
            sr[c][e] = pb;
          }
        } else if (cls[c] == 1) {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            uint32_t pb = __float_as_uint(fast_exp2(fmaf(__uint_as_float(sr[c][e]), sc, neg_shift))) & 0xffffe000u;
            pb = ((vmask[c] >> e) & 1u) ? pb : 0u;
            ls[e & 3] += __uint_as_float(pb);
            sr[c][e] = pb;
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) sr[c][e] = 0u;
        }
        tmem_st32(tS + c * 32, sr[c]);
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(bar(B_PREADY + sb));
      l_run += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      if (it == 0 && !early_look) prefetch_old_row();
    }
    const bool fresh = (l_in0 == 0.f) && (fabsf(o_first) <= 3.402823466e38f);  // the incoming state of this row is empty
    // ---- epilogue: O row from TMEM, normalised and merged with the caller's (m, l, O) ----
    if (nx > 0) {  // uniform over the softmax group, so the group barriers below are safe
      // both tile parities: the PVs of the last two tiles
      if (ok && nx > 1)
        ok = __all_sync(kFullMask, mbar_wait(bar(B_OREADY + x * 2 + ((nx - 2) & 1)), (uint32_t)(((nx - 2) >> 1) & 1),
                                             abort_flag, err, 304));
      ok = ok && __all_sync(kFullMask, mbar_wait(bar(B_OREADY + x * 2 + ((nx - 1) & 1)), (uint32_t)(((nx - 1) >> 1) & 1),
                                                 abort_flag, err, 303));
      // The epilogue uses a group barrier, which has no timeout: agree first (barrier + AND-reduction that
      // every thread of the group executes) that no warp of the group gave up on a wait.
      {
        uint32_t all_ok;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.and.pred q, %2, 128, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
            : "=r"(all_ok)
            : "r"((uint32_t)ok), "r"(1 + x)
            : "memory");
        ok = all_ok != 0;
      }
      if (ok) {
        tc_fence_after();
        const bool partial_out = (prm.mode == 2);
        // mode 2 writes a partial state for every real row (also rows with no key in this range);
        // the other modes touch a row only if it attended to something and is theirs to write
        const bool store = partial_out ? row_valid : (row_valid && l_run > 0.f && !listed);
        // Per-row coefficients of  O_out = ca * O_in + cb * O_tmem  (state in natural-log units, as the
        // gather path; l is re-expressed against the true maximum, O in TMEM is relative to `shift`).
        float ca = 0.f, cb = 0.f;
        if (store && !partial_out) {
          const int64_t rl = prm.r + uq * prm.s - prm.row_begin;  // shard-local row
          const float rel = fast_exp2(shift - m_true);
          const float l_loc = l_run * rel;
          const float m_loc = m_true * 0.6931471805599453f;
          const float m_in = m_in0, l_in = l_in0;  // read in the prologue
          const float m_o = fmaxf(m_in, m_loc);
          const float a = l_in * fast_exp2((m_in - m_o) * kLog2e);
          const float bt = fast_exp2((m_loc - m_o) * kLog2e);
          const float l_o = fmaf(l_loc, bt, a);
          const float inv = 1.0f / l_o;
          ca = a * inv;
          cb = bt * rel * inv;
          m_out[rl] = m_o;
          l_out[rl] = l_o;
        } else if (store) {
          // partial state of this key range: un-normalised O relative to the range's own maximum, then m, l
          float* part = prm.partials + ((size_t)uq * prm.n_split + blockIdx.y) * (D + 4);
          if (l_run > 0.f) {
            cb = fast_exp2(shift - m_true);
            part[D] = m_true * 0.6931471805599453f;
            part[D + 1] = l_run * cb;
          } else {
            cb = 0.f;
            part[D] = neg_inf();
            part[D + 1] = 0.f;
          }
        }
        constexpr int LPR = D / 4;  // float4 chunks (= lanes) per row
        uint8_t* stage = smem + P::kOffQ + x * P::kChunks * P::kQChunkBytes;
        // A sub-tile whose rows all carry an empty incoming state (the usual first call on a state) needs no merge:
        // cb * O_tmem IS the output. It is staged in the layout of the Q tile it replaces (32-column boxes of 128
        // rows, 128-byte swizzle) and leaves as D/32 bulk tensor stores issued by one thread: the per-thread path below
        // moves a 128 x D tile as 128 row-sized store instructions per warp, which the SM's store path takes at about
        // 32 bytes per cycle -- a fifth of a short CTA's life. Rows past the end of the shard are clipped by the tensor
        // map; a sub-tile with a row that must not be written (a listed row, a row without keys) or that has old state
        // takes the per-thread path.
        bool bulk = false;
        if (prm.tma_store && !partial_out) {
          uint32_t all_plain;
          asm volatile(
              "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.and.pred q, %2, 128, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
              : "=r"(all_plain)
              : "r"((uint32_t)(!row_valid || (store && fresh))), "r"(1 + x)
              : "memory");
          bulk = all_plain != 0;
        }
        if (bulk) {
          uint32_t ob[32];
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            tmem_ld32(tO + c * 32, ob);
            tc_wait_ld();
            uint8_t* box = stage + c * P::kQChunkBytes + (size_t)row * 128;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              float4 v4 = make_float4(cb * __uint_as_float(ob[4 * e + 0]), cb * __uint_as_float(ob[4 * e + 1]),
                                      cb * __uint_as_float(ob[4 * e + 2]), cb * __uint_as_float(ob[4 * e + 3]));
              *reinterpret_cast<float4*>(box + ((e ^ (row & 7)) << 4)) = v4;
            }
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the stores above, to the bulk-copy engine
          asm volatile("bar.sync %0, 128;" ::"r"(1 + x) : "memory");
          if (row == 0) {
            const int32_t yq = (int32_t)(uq0 - prm.u_q_first) + 128 * x;
#pragma unroll
            for (int c = 0; c < D / 32; ++c)
              asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(
                               reinterpret_cast<uint64_t>(&tmO)),
                           "r"(c * 32), "r"(yq), "r"(zs), "r"(sbase + P::kOffQ + (x * P::kChunks + c) * P::kQChunkBytes)
                           : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // shared memory is read out before the CTA ends
          }
        } else {
        // Stage cb * O_tmem in shared memory (this sub-tile's Q region is dead: all its S MMAs completed
        // before the last PV), 16-byte chunks XOR-swizzled by the row so that both the row-per-thread
        // writes here and the row-per-lane-group reads below spread over the banks.
        const uint32_t store_mask = __ballot_sync(kFullMask, store);  // bit = row of this warp (lane <-> row)
        const uint32_t read_mask = __ballot_sync(kFullMask, store && !fresh);  // rows whose old O row counts
        {
          uint32_t ob[32];
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            tmem_ld32(tO + c * 32, ob);
            tc_wait_ld();
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const int ch = c * 8 + e;
              float4 v4 = make_float4(cb * __uint_as_float(ob[4 * e + 0]), cb * __uint_as_float(ob[4 * e + 1]),
                                      cb * __uint_as_float(ob[4 * e + 2]), cb * __uint_as_float(ob[4 * e + 3]));
              *reinterpret_cast<float4*>(stage + (size_t)row * (D * 4) + ((ch ^ (row & (LPR - 1))) << 4)) = v4;
            }
          }
        }
        __syncwarp();  // every warp reads back only the 32 rows it staged itself
        // Coalesced read-modify-write of the caller's O rows: LPR lanes cover one row (D*4 contiguous bytes).
        constexpr int RPI = 32 / LPR;    // rows per warp instruction
        constexpr int NIT = 32 / RPI;    // instructions for this warp's 32 rows
        const int wrow0 = (warp & 3) * 32, sub = lane % LPR;
        if (partial_out) {
#pragma unroll 4
          for (int i = 0; i < NIT; ++i) {
            const int rw = i * RPI + lane / LPR, r = wrow0 + rw;
            if ((store_mask >> rw) & 1u) {
              float* part = prm.partials + ((size_t)(uq0 + 128 * x + r) * prm.n_split + blockIdx.y) * (D + 4);
              *reinterpret_cast<float4*>(part + sub * 4) =
                  *reinterpret_cast<const float4*>(stage + (size_t)r * (D * 4) + ((sub ^ (r & (LPR - 1))) << 4));
            }
          }
        } else {
          // Eight rows-per-instruction steps at a time: enough old rows in flight when they have to be read, and a loop
          // body small enough to stay in the instruction cache (the epilogue runs once per CTA; fully unrolled it was
          // a few thousand cold instructions, and instruction fetch showed among the stalls of short CTAs).
          constexpr int NB = (NIT < 8) ? NIT : 8;
#pragma unroll 1
          for (int i0 = 0; i0 < NIT; i0 += NB) {
            float4 oin[NB];
#pragma unroll
            for (int k = 0; k < NB; ++k) {
              const int rw = (i0 + k) * RPI + lane / LPR, r = wrow0 + rw;
              oin[k] = make_float4(0.f, 0.f, 0.f, 0.f);
              if ((read_mask >> rw) & 1u) {
                const int64_t rl = prm.r + (uq0 + 128 * x + r) * prm.s - prm.row_begin;
                oin[k] = *reinterpret_cast<const float4*>(O_out + (size_t)rl * D + sub * 4);
              }
            }
#pragma unroll
            for (int k = 0; k < NB; ++k) {
              const int rw = (i0 + k) * RPI + lane / LPR, r = wrow0 + rw;
              const float car = __shfl_sync(kFullMask, ca, rw);  // the row's coefficient lives in the lane that owns the row
              if ((store_mask >> rw) & 1u) {
                const int64_t rl = prm.r + (uq0 + 128 * x + r) * prm.s - prm.row_begin;
                const float4 t =
                    *reinterpret_cast<const float4*>(stage + (size_t)r * (D * 4) + ((sub ^ (r & (LPR - 1))) << 4));
                float4 o;
                o.x = fmaf(car, oin[k].x, t.x);
                o.y = fmaf(car, oin[k].y, t.y);
                o.z = fmaf(car, oin[k].z, t.z);
                o.w = fmaf(car, oin[k].w, t.w);
                *reinterpret_cast<float4*>(O_out + (size_t)rl * D + sub * 4) = o;
              }
            }
          }
        }
        }  // per-thread path
      }
    }
  }

  // ---- common exit: everyone is done with TMEM before it is released ----
  tc_fence_before();
  __syncthreads();
  // started early beside its predecessor: completion order (and with it everything later in the stream) must
  // still see the predecessor finished
  if ((prm.overlap & 2) && threadIdx.x == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
  if (warp == W_TMA) {
    tc_fence_after();
    if (*abort_flag && lane == 0) {
      // give copies that may still be in flight time to land before the CTA's shared memory is reused
      const uint64_t t0 = globaltimer();
      while (globaltimer() - t0 < 2000000ull) {
      }
    }
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(P::kTmemCols) : "memory");
  }
}

}  // namespace tile
}  // namespace spfa
