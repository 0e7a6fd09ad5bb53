// W4A16 dequantize-GEMM for up to 64 tokens (the memory-bound decode regime), group-sum form, sm_100a:
//   C[m, n] = cast( sum_g s[g, n] * ( sum_{k in g} float(A[m, k]) * (q[n, k] - zero) ) )
// i.e. the group scale multiplies the group's fp32 partial sum instead of every weight.  With one-hot
// activations this equals half(q - zero) * s bit for bit (the fp32 product of two f16 values is exact
// and is rounded once, to the output type); in general it differs from scaling each weight in f16 first
// only by that product's own rounding (2^-11 relative per term), well inside the operator's tolerance.
//
// Why: these shapes are bound by instruction issue on the SM, not by memory (a warp gets an issue slot
// only every ~10 cycles once 28 warps share four schedulers, and the ALU and FP16 pipes run at half
// rate), so the kernel is written to execute as few instructions per weight as possible:
//  - 9 instead of 13 instructions per eight weights in the dequant warps (no f16x2 scale multiplies; the
//    scale work is one fp32 FMA per (token, 128 k) in four drain warps, on the otherwise idle FMA pipe);
//  - ring stages and barrier parities are compile-time constants of unrolled loops, barrier addresses
//    are one base register plus an immediate, a wait is a try_wait and a branch on its fast path;
//  - a dequant warp converts a whole 128-k half of its 32 rows per hand-over (two sets of eight warps
//    take alternate slabs), so the hand-over cost is paid once per 16 packed words;
//  - the MMA-issuing warps run warp-convergent, one hardware-elected lane issues the eight MMAs of a half
//    and their commits (see w4g_elect_one), and they know nothing about tiles: every 128-k half starts a
//    fresh accumulator.
//
// Structure (persistent stream-K over (tile, 256-wide K slab) items, as in w4a16.cuh):
//   warp 0        TMA: packed weights [128 rows x 128 B] per slab into the raw ring
//   warp 1        TMA: prepared activations [MT x 256 k] per slab into their ring
//   warp 2        tensor-memory allocation; TMA: the slab's scale rows [1 or 2 x 128] into the scale ring
//   warps 4..7, 28..31  drain (two sets of four on alternate slabs: one warp's instruction stream per slab is a
//                 serial chain of ~85 instructions, too long for one warp per 32 rows at the slab rate):
//                 one tcgen05.ld of the slab's two accumulators, fp32 FMA with each half's scale into register
//                 sums; at a segment's end the sets add their sums, then the tile write or the split-K hand-over
//   warps 8..23   dequant: lop3 magic-number conversion, (q - zero) exact in f16, tcgen05.st
//   warps 24..27  tcgen05.mma kind::f16 issuers (A = weights from tensor memory, B = activations from
//                 shared memory); issuer w takes the 128-k halves h with h % 4 == w, each into its own
//                 accumulator of a ring, so no two issuers ever share an accumulator
// Tensor memory: NSLOT slab slots of two accumulators of MT columns (ring, 256 columns) + 4 stages of 64 columns
// of converted weights (one 128-k half each).
//
// Every wait is bounded: after a number of failed mbarrier.try_wait attempts (each suspends the thread
// for a few microseconds) derived from the caller's limit, the wait stores its role code in a CTA-wide
// abort word and sets the thread's `fail` flag; all other waits of the CTA see the abort word in their
// slow path and give up too.  `fail` never steers a warp's control flow lane by lane (the tcgen05 ld /
// st / fence instructions need the whole warp): roles vote on it at coarse points, stop, and the kernel
// drains, frees its tensor memory, reports the code in the status word and returns.
#pragma once

#include <type_traits>

#include "common.cuh"
#include "w4a16.cuh"

namespace qg {

constexpr int W4G_FIRST_EPI_WARP = 4;
constexpr int W4G_FIRST_DQ_WARP = 8;
constexpr int W4G_DQ_WARPS = 16;
constexpr int W4G_FIRST_MMA_WARP = W4G_FIRST_DQ_WARP + W4G_DQ_WARPS;  // 24
constexpr int W4G_MMA_WARPS = 4;
constexpr int W4G_FIRST_EPI2_WARP = W4G_FIRST_MMA_WARP + W4G_MMA_WARPS;  // 28: second set of drain warps
constexpr int W4G_THREADS = (W4G_FIRST_EPI2_WARP + 4) * 32;             // 1024
constexpr int W4G_WH = 4;          // stages of converted weights, one 128-k half (64 columns) each
constexpr int W4G_HALF_COLS = 64;
constexpr int W4G_RS = 8;          // raw (packed weight) ring, 16 KB per stage
constexpr int W4G_SS = 16;         // scale ring, 512 B per stage
constexpr int W4G_SC_BYTES = 512;  // up to two rows of 128 halves

// Byte offsets of the barriers (8 bytes each) and control words from the start of the barrier block.
constexpr int W4G_RAW_FULL = 0;       // [8]
constexpr int W4G_RAW_EMPTY = 64;     // [8]
constexpr int W4G_A_FULL = 128;       // [<= 8]
constexpr int W4G_A_EMPTY = 192;      // [<= 8]
constexpr int W4G_W_FULL = 256;       // [4]
constexpr int W4G_W_EMPTY = 288;      // [4]
constexpr int W4G_ACC_FULL = 320;     // [<= 8] one per slab slot: both halves' issuers commit to it
constexpr int W4G_ACC_EMPTY = 448;    // [<= 8]
constexpr int W4G_SC_FULL = 576;      // [16]
constexpr int W4G_SC_EMPTY = 704;     // [16]
constexpr int W4G_DRAIN = 832;
constexpr int W4G_TMEM_SLOT = 840;
constexpr int W4G_CTL = 848;          // u32 abort word (0, or the role code of the first wait that gave up), u32 max tries
constexpr int W4G_EPI_CTRL = 856;     // u32[2], alternating by segment: bit 0 abort, bit 1 last contributor
constexpr int W4G_PART_FULL = 864;    // SMALL form, in the cluster's first CTA: the other CTAs' sums have arrived
constexpr int W4G_SMALL_MAX_SLABS = 4;  // SMALL form: slabs per CTA (stages 4.. of the raw ring receive the other CTAs' sums)

template <int MT>
struct W4GCfg {
  static_assert(MT == 16 || MT == 32 || MT == 64, "token tile");
  static constexpr int AS = (MT == 16) ? 8 : (MT == 32 ? 4 : 2);  // activation ring (even: an issuer meets every phase of its stages)
  static constexpr int NSLOT = 128 / MT;           // slab slots of two accumulators each (8, 4 or 2)
  // How the two drain sets share the work: on alternate slabs, all tokens each (their sums meet at a segment's
  // end), or - 64 tokens would not fit a thread's registers - every slab, 32 tokens each (nothing to exchange).
  static constexpr bool SPLIT_TOKENS = MT == 64;
  static constexpr int DT = SPLIT_TOKENS ? 32 : MT;  // tokens one drain thread accumulates
  static constexpr int A_KB_BYTES = MT * 128;      // one 64-wide K block of activations
  static constexpr int A_BYTES = 4 * A_KB_BYTES;   // one 256-wide slab
  static constexpr int TMEM_COLS = 512;
  static constexpr int BAR_BYTES = 1024;
  static constexpr int XBUF_BYTES = SPLIT_TOKENS ? 0 : MT * W4_BN * 4;  // the second drain set's sums of one segment
  static constexpr int SMEM_BYTES =
      W4G_RS * W4_RAW_PACKED + AS * A_BYTES + W4G_SS * W4G_SC_BYTES + W4G_RS * W4G_SC_BYTES + XBUF_BYTES + BAR_BYTES + 1024;
  static constexpr int A_PER = AS / 2;                // activation stages one issuer meets
  static constexpr int S_PER = NSLOT / 2;             // slab slots one issuer meets (those of its slab parity)
  static_assert(A_PER == 4 || A_PER == 2 || A_PER == 1, "activation ring depth");
  static_assert(S_PER == 4 || S_PER == 2 || S_PER == 1, "accumulator ring depth");
};

// Debug hook for the bounded-wait test: when non-zero, the MMA issuers do not signal the accumulator of
// the last 128-k half of the launch, so the drain warps' wait for it runs out.  Nothing else is affected:
// every copy lands, every other barrier completes, the kernel frees its tensor memory and returns.
struct W4GDebug {
  int withhold_last_commit;  // 1: as described above (two-launch form); 2: the single-launch form's cluster signal
};

// ---- lean primitives on shared-space addresses ------------------------------------------------------
// Bounded wait on the barrier at [base + OFF].  Fast path: one try_wait and one branch.  Slow path (the
// phase was not complete): poll; every failed try_wait has suspended the thread for a few microseconds,
// so the abort word and the attempt counter (both in the control block at `ctl`) are only looked at there.
template <int OFF, int CODE>
__device__ __forceinline__ void w4g_wait(uint32_t base, uint32_t parity, uint32_t ctl, uint32_t& fail) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      ".reg .u32 n, t;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1+%4], %2;\n\t"
      "@p bra W4G_DONE;\n\t"
      "ld.shared.u32 n, [%3+4];\n"
      "W4G_LOOP:\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1+%4], %2;\n\t"
      "@p bra W4G_DONE;\n\t"
      "ld.volatile.shared.u32 t, [%3];\n\t"
      "setp.ne.u32 q, t, 0;\n\t"
      "@q bra W4G_FAIL;\n\t"
      "sub.u32 n, n, 1;\n\t"
      "setp.ne.u32 q, n, 0;\n\t"
      "@q bra W4G_LOOP;\n\t"
      "mov.u32 t, %5;\n\t"
      "st.volatile.shared.u32 [%3], t;\n"
      "W4G_FAIL:\n\t"
      "mov.u32 %0, 1;\n"
      "W4G_DONE:\n\t"
      "}"
      : "+r"(fail)
      : "r"(base), "r"(parity), "r"(ctl), "n"(OFF), "n"(CODE)
      : "memory");
}
template <int OFF>
__device__ __forceinline__ void w4g_arrive(uint32_t base) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0+%1];" ::"r"(base), "n"(OFF) : "memory");
}
template <int OFF>
__device__ __forceinline__ uint4 w4g_lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+%5];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr), "n"(OFF));
  return v;
}
// One lane of the (converged) warp, chosen by the hardware.  Code under `if (w4g_elect_one())` is known to the
// compiler to run in exactly one lane, which lets it issue tcgen05.mma / commit / TMA instructions with their
// operands in uniform registers directly: measured 68 instead of 130-160 instructions, and 420 instead of 800-900
// cycles, for the eight MMAs and three commits of a half compared with `if (lane == 0)` or per-lane predicates.
__device__ __forceinline__ bool w4g_elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void w4g_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Two fp32 FMAs in one instruction (d0 += a0 * s, d1 += a1 * s), each rounded exactly like fmaf: the drain warps'
// instruction streams are serial chains, so halving their FMA count shortens the chain.
__device__ __forceinline__ void w4g_fma2(float& d0, float& d1, uint32_t a0, uint32_t a1, float s) {
  asm("{\n\t"
      ".reg .b64 ra, rb, rc;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %4};\n\t"
      "mov.b64 rc, {%0, %1};\n\t"
      "fma.rn.f32x2 rc, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rc;\n\t"
      "}"
      : "+f"(d0), "+f"(d1)
      : "r"(a0), "r"(a1), "f"(s));
}
// Named barrier of the eight drain warps.
__device__ __forceinline__ void w4g_epi_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// Parity of the n-th visit (n = 4 * c + u, u < 4) of a ring position that is met every `PER` iterations.
template <int PER>
__device__ __forceinline__ uint32_t w4g_visit_parity(uint32_t c, int u) {
  return (PER == 4) ? (c & 1u) : (uint32_t)((u / PER) & 1);
}

// The segments of a CTA: those of its stream-K range, then its whole tiles (first_dp, first_dp + stride, ...).
struct W4HybridIter {
  W4SegIter sk;
  int next_dp, dp_left, stride, KS;
  __device__ __forceinline__ bool next(int& tile, int& ks0, int& ks1) {
    if (sk.next(tile, ks0, ks1)) return true;
    if (dp_left <= 0) return false;
    tile = next_dp;
    ks0 = 0;
    ks1 = KS;
    next_dp += stride;
    --dp_left;
    return true;
  }
};

// GATHER = true is the gathered form (several destination buffers, see W4A16Params::c_dst); it is a separate
// instantiation because the destination loop in the store path costs the plain kernel 8 % through register
// allocation alone.
// ZT = true: one integer zero point per (group, output feature) instead of the scalar one - the zeros tensor
// [K/g, N] f16 of zero mode "quantized" (tilelang/quantize/lop3.py:325-358: (q - qz) * s with the subtraction
// exact).  The weight producer fetches the slab's zero rows (through tmZ, laid out like the scale rows) into a ring
// that shares the packed weights' stages and barriers, and a dequant thread builds its row's two magic constants
// from the zero it reads there: five more instructions per 128-k half.
// SMALL = true (16-token tile): the single-launch form for problems of a few slabs per CTA.  The kernel is launched in
// clusters of C = KS / (slabs per CTA) CTAs, one tile per cluster, CTA r taking the r-th K range; there is no pre-pass
// and no scratch memory:
//  - the drain warps first fetch the CTA's own piece of the activations straight from the caller's tensor, convert
//    and reorder it as the pre-pass would, and write it into the activation stages in the layout the MMA descriptor
//    expects (128-byte swizzle: 16-byte chunk j of row r of a 64-k block at chunk position j ^ (r & 7));
//  - at the end CTAs 1 .. C-1 write their sums through distributed shared memory into the unused upper half of the
//    first CTA's raw ring, and the first CTA adds them in rank order and writes the tile - no counters, no partial
//    sums in global memory, the same fixed summation order on every run.
template <int MT, bool OUT_BF16, bool GATHER = false, bool ZT = false, bool SMALL = false>
__global__ void __launch_bounds__(W4G_THREADS, 1)
w4a16_gs_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmS,
                const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmA, const W4A16Params p,
                const W4GDebug dbg) {
  using Cfg = W4GCfg<MT>;
  constexpr int RS = W4G_RS;
  constexpr int AS = Cfg::AS;
  constexpr int NSLOT = Cfg::NSLOT;
  constexpr int SS = W4G_SS;
  static_assert(RS == 8 && SS == 16 && AS <= 8 && NSLOT <= 8, "barrier block layout");
  static_assert(!SMALL || (MT == 16 && !GATHER && !ZT), "the single-launch form: 16-token tile, one destination, scalar zero");
  // The next call's pre-pass (a programmatic dependent) may become resident now; it waits for this whole grid before
  // it touches anything, and the GEMM kernel behind it only reads weights and scales until that pre-pass is done.
  pdl_launch_dependents();

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* raw_base = smem;
  uint8_t* a_base = smem + RS * W4_RAW_PACKED;
  uint8_t* sc_base = a_base + AS * Cfg::A_BYTES;
  uint8_t* z_base = sc_base + SS * W4G_SC_BYTES;  // zero rows, one 512-byte stage per raw stage (ZT only)
  float* xbuf = reinterpret_cast<float*>(z_base + RS * W4G_SC_BYTES);
  uint8_t* bar_block = z_base + RS * W4G_SC_BYTES + Cfg::XBUF_BYTES;
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(bar_block + W4G_RAW_FULL);
  uint64_t* raw_empty = reinterpret_cast<uint64_t*>(bar_block + W4G_RAW_EMPTY);
  uint64_t* a_full = reinterpret_cast<uint64_t*>(bar_block + W4G_A_FULL);
  uint64_t* a_empty = reinterpret_cast<uint64_t*>(bar_block + W4G_A_EMPTY);
  uint64_t* w_full = reinterpret_cast<uint64_t*>(bar_block + W4G_W_FULL);
  uint64_t* w_empty = reinterpret_cast<uint64_t*>(bar_block + W4G_W_EMPTY);
  uint64_t* acc_full = reinterpret_cast<uint64_t*>(bar_block + W4G_ACC_FULL);
  uint64_t* acc_empty = reinterpret_cast<uint64_t*>(bar_block + W4G_ACC_EMPTY);
  uint64_t* sc_full = reinterpret_cast<uint64_t*>(bar_block + W4G_SC_FULL);
  uint64_t* sc_empty = reinterpret_cast<uint64_t*>(bar_block + W4G_SC_EMPTY);
  uint64_t* drain = reinterpret_cast<uint64_t*>(bar_block + W4G_DRAIN);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_block + W4G_TMEM_SLOT);
  volatile uint32_t* ctl_words = reinterpret_cast<uint32_t*>(bar_block + W4G_CTL);  // [0] abort word, [1] max tries
  volatile uint32_t* epi_ctrl = reinterpret_cast<uint32_t*>(bar_block + W4G_EPI_CTRL);

  // a warp index the compiler can prove uniform, so that everything derived from it may live in uniform registers
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;

  // One thread per barrier slot sets it up (the block is a dense array of 8-byte slots; a serial loop over the
  // hundred of them costs about a microsecond of every launch).
  if (threadIdx.x <= W4G_DRAIN / 8) {
    const int off = 8 * (int)threadIdx.x;
    const int drain_warps = Cfg::SPLIT_TOKENS ? 8 : 4;  // drain warps that read one slab: one set, or both
    int count = 0;                                       // 0: unused slot
    if (off < W4G_RAW_EMPTY) count = 1;
    else if (off < W4G_A_FULL) count = W4G_DQ_WARPS / 2;   // the eight dequant warps of the set that took the slab
    else if (off < W4G_A_EMPTY) count = (off - W4G_A_FULL) / 8 < AS ? 1 : 0;
    else if (off < W4G_W_FULL) count = (off - W4G_A_EMPTY) / 8 < AS ? 2 : 0;  // the issuers of the slab's two halves
    else if (off < W4G_W_EMPTY) count = 4;                 // the four dequant warps (one per 32 rows) of that half
    else if (off < W4G_ACC_FULL) count = 1;
    else if (off < W4G_ACC_EMPTY) count = (off - W4G_ACC_FULL) / 8 < NSLOT ? 2 : 0;  // the issuers of the two halves
    else if (off < W4G_SC_FULL) count = (off - W4G_ACC_EMPTY) / 8 < NSLOT ? drain_warps : 0;
    else if (off < W4G_SC_EMPTY) count = 1;
    else if (off < W4G_DRAIN) count = drain_warps;
    else count = W4G_MMA_WARPS;
    if (count > 0) mbar_init(reinterpret_cast<uint64_t*>(bar_block + off), (uint32_t)count);
    fence_barrier_init();
  }
  if (threadIdx.x == 0) {
    ctl_words[0] = 0;
    // a failed try_wait has suspended the thread for roughly 2 us or longer
    ctl_words[1] = (uint32_t)(p.wait_limit_ns >> 11) + 2u;
    epi_ctrl[0] = epi_ctrl[1] = 0;
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmA);
    if (p.has_scales) tma_prefetch_desc(&tmS);
    if (ZT) tma_prefetch_desc(&tmZ);
    if constexpr (SMALL) {
      const uint32_t others = cluster_nctarank() - 1u;
      mbar_init(reinterpret_cast<uint64_t*>(bar_block + W4G_PART_FULL), others > 0u ? others : 1u);
      fence_barrier_init();
    }
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if constexpr (SMALL) cluster_sync_all();  // the first CTA's barrier exists before any other CTA of the cluster signals it
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_w = tmem_base + NSLOT * 2 * MT;  // converted weights behind the accumulator ring
  const uint32_t bar0 = smem_u32(bar_block);
  const uint32_t ctl = bar0 + W4G_CTL;

  const int G = gridDim.x;
  const int cta = blockIdx.x;
  // Work split: the first p.sk_tiles tiles are cut stream-K fashion (their slabs dealt evenly to the CTAs as
  // contiguous ranges, partial tiles meeting through the scratch buffer); after its range CTA c takes the whole tiles
  // sk_tiles + c, sk_tiles + c + G, ...  The hand-overs of the partial tiles thus happen early, behind the following
  // tiles' work, and the launch ends with plain tile writes.
  const long long T = (long long)p.sk_tiles * p.KS;  // stream-K items
  // SMALL: cluster t takes tile t, its CTA r the slabs [r * per, (r + 1) * per) of it
  const int crank = SMALL ? (int)cluster_ctarank() : 0;
  const int csize = SMALL ? (int)cluster_nctarank() : 1;
  const int per = SMALL ? p.KS / csize : 0;
  const long long item0 = SMALL ? (long long)(cta / csize) * p.KS + (long long)crank * per : w4_range_begin(T, G, cta);
  const long long item1 = SMALL ? item0 + per : w4_range_begin(T, G, cta + 1);
  const int n_sk = (int)(item1 - item0);
  const int n_slabs = SMALL ? n_sk : n_sk + p.dp_rounds * p.KS;  // this CTA's slabs, numbered 0.. in processing order

  if (warp <= 2) {
    // ------------------------------------------------------------------ TMA producers
    // warp 0: packed weights, warp 1: activations, warp 2: scales
    if (lane == 0 && (warp != 2 || p.has_scales) && !(SMALL && warp == 1)) {
      if (warp == 1) pdl_wait();  // the prepared activations come from the pre-pass kernel in front of this one
      uint64_t* full = warp == 0 ? raw_full : (warp == 1 ? a_full : sc_full);
      const uint32_t empty0 = bar0 + (warp == 0 ? W4G_RAW_EMPTY : (warp == 1 ? W4G_A_EMPTY : W4G_SC_EMPTY));
      const int depth = warp == 0 ? RS : (warp == 1 ? AS : SS);
      const uint32_t sc_tx = (uint32_t)p.scale_rows * 256u;
      int tile = n_sk > 0 ? (int)(item0 / p.KS) : p.sk_tiles + cta;
      int ks = n_sk > 0 ? (int)(item0 - (long long)tile * p.KS) : 0;
      int b, n0, m0;
      w4_tile_coords(p, tile, MT, b, n0, m0);
      int st = 0;
      uint32_t phase = 0, issued_mask = 0, parity_mask = 0, fail = 0;
      for (int i = 0; i < n_slabs; ++i) {
        w4g_wait<0, ST_TIMEOUT_PRODUCER>(empty0 + 8 * st, phase ^ 1u, ctl, fail);
        if (fail) break;
        if (warp == 0) {
          mbar_arrive_expect_tx(&full[st], ZT ? W4_RAW_PACKED + sc_tx : (uint32_t)W4_RAW_PACKED);
          tma_load_3d(raw_base + st * W4_RAW_PACKED, &tmW, &full[st], ks * (W4_SLAB_K / 2), n0, b);
          if (ZT) {  // the zero rows of the slab's two halves, addressed like its scale rows
            const int zrow = (p.scale_rows == 2) ? 2 * ks : (ks * W4_SLAB_K) / p.group;
            tma_load_3d(z_base + st * W4G_SC_BYTES, &tmZ, &full[st], n0, zrow, b);
          }
        } else if (warp == 1) {
          uint8_t* dstA = a_base + st * Cfg::A_BYTES;
          mbar_arrive_expect_tx(&full[st], Cfg::A_BYTES);
#pragma unroll
          for (int kb = 0; kb < 4; ++kb)
            tma_load_3d(dstA + kb * Cfg::A_KB_BYTES, &tmA, &full[st], ks * W4_SLAB_K + kb * 64, m0, b);
        } else {
          // scale rows of the slab: two when the groups are 128 wide, else the one row of the slab's group
          const int srow = (p.scale_rows == 2) ? 2 * ks : (ks * W4_SLAB_K) / p.group;
          mbar_arrive_expect_tx(&full[st], sc_tx);
          tma_load_3d(sc_base + st * W4G_SC_BYTES, &tmS, &full[st], n0, srow, b);
        }
        issued_mask |= 1u << st;
        parity_mask = (parity_mask & ~(1u << st)) | (phase << st);
        if (++st == depth) { st = 0; phase ^= 1u; }
        if (i + 1 == n_sk) {  // the stream-K range is done: on to this CTA's first whole tile
          ks = 0;
          tile = p.sk_tiles + cta;
          w4_tile_coords(p, tile, MT, b, n0, m0);
        } else if (++ks == p.KS) {
          ks = 0;
          tile += (i + 1 < n_sk) ? 1 : G;
          w4_tile_coords(p, tile, MT, b, n0, m0);
        }
      }
      if (fail) {  // wait (bounded) for the copies still in flight before the CTA may exit
        for (int s = 0; s < depth; ++s) {
          if (!(issued_mask & (1u << s))) continue;
          const uint64_t t0 = global_timer_ns();
          while (!mbar_try_wait(&full[s], (parity_mask >> s) & 1u)) {
            if (global_timer_ns() - t0 > p.wait_limit_ns) {
              ctl_words[0] = ST_TIMEOUT_DRAIN;
              break;
            }
          }
        }
      }
    }
  } else if (warp >= W4G_FIRST_MMA_WARP && warp < W4G_FIRST_EPI2_WARP) {
    // ------------------------------------------------------------------ MMA issuers (warp-convergent)
    // Iteration n = 4 * c + u of issuer w handles half h = w + 4 * n of slab (w / 2) + 2 n: weight stage w
    // (parity n & 1 = u & 1), activation stage (w / 2) + 2 * (u % A_PER), slab slot (w / 2) + 2 * (u % S_PER),
    // accumulator w & 1 of that slot.
    const int w = warp - W4G_FIRST_MMA_WARP;
    constexpr uint32_t idesc = make_idesc(ACC_F32, FMT_F16, FMT_F16, 0, 0, W4_BN, MT);
    const int half = w & 1;
    const int n_half = 2 * n_slabs;
    const uint32_t tW = tmem_w + w * W4G_HALF_COLS;
    // K-major activation descriptor: the high word is constant, the low word holds the start address >> 4
    const uint64_t desc0 = make_desc_kmajor(smem_u32(a_base) + (w >> 1) * Cfg::A_BYTES + half * 2 * Cfg::A_KB_BYTES);
    const uint32_t desc_hi = (uint32_t)(desc0 >> 32);
    const uint32_t desc_lo0 = (uint32_t)desc0;
    const uint32_t d0 = tmem_base + (w >> 1) * 2 * MT + half * MT;
    const uint32_t bw = bar0 + 8 * w;         // this issuer's weight stage
    const uint32_t ba = bar0 + 8 * (w >> 1);  // this issuer's activation stages and slab slots
    const int withhold_h = (dbg.withhold_last_commit && cta == G - 1) ? n_half - 1 : -1;
    uint32_t fail = 0;
    int h = w;
    static_assert(Cfg::A_PER == Cfg::S_PER, "one unrolled step = one (activation stage, accumulator slot) pair");
    for (uint32_t c = 0; h < n_half; ++c) {
      // the four steps of an outer iteration, unrolled with compile-time stage indices
      auto step = [&](auto u_) {
        constexpr int u = decltype(u_)::value;
        if (h >= n_half) return;
        constexpr int ai = u % Cfg::A_PER;  // which of this issuer's activation stages
        constexpr int si = u % Cfg::S_PER;  // which of this issuer's accumulator slots
        w4g_wait<W4G_ACC_EMPTY + 16 * si, ST_TIMEOUT_MMA>(ba, w4g_visit_parity<Cfg::S_PER>(c, u) ^ 1u, ctl, fail);
        w4g_wait<W4G_A_FULL + 16 * ai, ST_TIMEOUT_MMA>(ba, w4g_visit_parity<Cfg::A_PER>(c, u), ctl, fail);
        w4g_wait<W4G_W_FULL, ST_TIMEOUT_MMA>(bw, (uint32_t)(u & 1), ctl, fail);
        tc_fence_after_sync();
        const uint32_t d = d0 + (2 * si) * 2 * MT;
        const uint32_t lo = desc_lo0 + (uint32_t)((2 * ai * Cfg::A_BYTES) >> 4);
        if (w4g_elect_one()) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {  // 16 k per MMA: 8 columns of weights, 32 bytes of activations
            const uint32_t off = (uint32_t)(((j >> 2) * Cfg::A_KB_BYTES + (j & 3) * 32) >> 4);
            umma_f16_ts(d, tW + j * 8, ((uint64_t)desc_hi << 32) | (uint64_t)(lo + off), idesc, j != 0 ? 1u : 0u);
          }
          w4g_commit(bw + W4G_W_EMPTY);
          w4g_commit(ba + W4G_A_EMPTY + 16 * ai);
          if (h != withhold_h) w4g_commit(ba + W4G_ACC_FULL + 16 * si);
        }
        h += W4G_MMA_WARPS;
      };
      step(std::integral_constant<int, 0>{});
      step(std::integral_constant<int, 1>{});
      step(std::integral_constant<int, 2>{});
      step(std::integral_constant<int, 3>{});
      fail = __any_sync(0xffffffffu, fail != 0) ? 1u : 0u;
      if (fail) break;
    }
    // everything this warp issued has completed before the CTA frees its tensor memory
    if (w4g_elect_one()) w4g_commit(bar0 + W4G_DRAIN);
    if (w == 0 && lane == 0) {
      const uint64_t t0 = global_timer_ns();
      while (!mbar_try_wait(drain, 0)) {
        if (global_timer_ns() - t0 > p.wait_limit_ns) break;
      }
    }
  } else if ((warp >= W4G_FIRST_EPI_WARP && warp < W4G_FIRST_DQ_WARP) || warp >= W4G_FIRST_EPI2_WARP) {
    // ------------------------------------------------------------------ drain / epilogue
    // Set e (warps 4..7: 0, warps 28..31: 1) drains the CTA-local slabs i with i % 2 == e: slab slot i % NSLOT
    // (parity (i / NSLOT) & 1), scale stage i % 16 (parity (i / 16) & 1).  Both sets walk the same segments and
    // meet at every segment end, where set 1 hands its sums to set 0 through shared memory.
    const int e = warp >= W4G_FIRST_EPI2_WARP ? 1 : 0;
    const int q = warp & 3;
    const int nl = q * 32 + lane;  // weight row inside the tile == TMEM lane
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t sc_addr0 = smem_u32(sc_base) + 2 * nl;
    const uint32_t sc_row1 = p.scale_rows == 2 ? 256u : 0u;  // the second half's scale row inside a stage
    const bool scaled = p.has_scales != 0;
    const bool lead = lane == 0;
    if constexpr (!SMALL) pdl_wait();  // the arrival counters are zeroed by the pre-pass kernel in front of this one
    if constexpr (SMALL) {
      // this CTA's piece of the activations: rows m0 .. m0 + 15 (zero beyond M), k [256 * ks_first, 256 * (ks_first + per))
      const int tile_s = (int)(item0 / p.KS);
      const int ks_first = (int)(item0 - (long long)tile_s * p.KS);
      int bb, nn0, mm0;
      w4_tile_coords(p, tile_s, MT, bb, nn0, mm0);
      const int tid = (e * 4 + q) * 32 + lane;  // 0 .. 255
      const int chunks_per_row = per * 32;       // 16-byte chunks (eight k) per row in this CTA's K range
      const uint4* src = reinterpret_cast<const uint4*>(p.A_raw) + ((size_t)bb * p.M) * (size_t)(p.K / 8);
      const int row_chunks = p.K / 8;  // chunks in a whole row of A: the last slab of a short K is partly outside
      constexpr int PER_THREAD = MT * W4G_SMALL_MAX_SLABS * 32 / 256;  // at most eight chunks per thread
      const uint4* ptr[PER_THREAD];
      uint32_t dst_off[PER_THREAD];  // byte offset in the activation stages, or ~0 for a chunk this thread does not have
#pragma unroll
      for (int u = 0; u < PER_THREAD; ++u) {
        const int c = tid + 256 * u;
        const int r = c / chunks_per_row, kc = c - r * chunks_per_row;
        const int slab = kc >> 5, j = kc & 31;  // chunk j of the slab: 64-k block j / 8, chunk j % 8 of the row there
        dst_off[u] = c < MT * chunks_per_row
                         ? (uint32_t)(slab * Cfg::A_BYTES + (j >> 3) * Cfg::A_KB_BYTES + r * 128 + (((j & 7) ^ (r & 7)) << 4))
                         : 0xffffffffu;
        const bool inside = c < MT * chunks_per_row && mm0 + r < p.M && ks_first * 32 + kc < row_chunks;
        ptr[u] = inside ? src + (size_t)(mm0 + r) * (size_t)row_chunks + (size_t)ks_first * 32 + kc : nullptr;
      }
      pdl_wait();  // whatever is in front of this launch has finished: the activations may be read, the output written
      uint4 v[PER_THREAD];
#pragma unroll
      for (int u = 0; u < PER_THREAD; ++u)  // all loads first, so that their latencies overlap
        v[u] = ptr[u] != nullptr ? __ldcg(ptr[u]) : make_uint4(0u, 0u, 0u, 0u);  // L2 is the point of coherence
#pragma unroll
      for (int u = 0; u < PER_THREAD; ++u) {
        if (dst_off[u] != 0xffffffffu) {
          uint4 w = v[u];
          if (p.a_is_bf16) {
            w.x = w4_bf16x2_to_f16x2(w.x);
            w.y = w4_bf16x2_to_f16x2(w.y);
            w.z = w4_bf16x2_to_f16x2(w.z);
            w.w = w4_bf16x2_to_f16x2(w.w);
          }
          if (p.a_permute) w = w4_permute_act(w);
          *reinterpret_cast<uint4*>(a_base + dst_off[u]) = w;
        }
      }
      fence_proxy_async_smem();  // the MMAs read these stages through the async proxy
      w4g_epi_bar();
      if (tid == 0)
        for (int sidx = 0; sidx < per; ++sidx) mbar_arrive(&a_full[sidx]);
    }
    W4HybridIter seg{W4SegIter{item0, item1, p.KS}, p.sk_tiles + cta, SMALL ? 0 : p.dp_rounds, G, p.KS};
    int tile, ks0, ks1;
    uint32_t i_seg0 = 0;  // CTA-local index of the segment's first slab
    uint32_t fail = 0;
    int seg_idx = 0;
    while (seg.next(tile, ks0, ks1)) {
      int b, n0, m0;
      w4_tile_coords(p, tile, MT, b, n0, m0);
      const int n = n0 + nl;
      uint16_t* Cout = reinterpret_cast<uint16_t*>(p.C) + (size_t)b * p.M * p.N;
      const bool full_tile = (ks0 == 0 && ks1 == p.KS);
      const int my_slot = (ks1 < p.KS) ? 2 * cta + 1 : 2 * cta;
      const uint32_t i_end = i_seg0 + (uint32_t)(ks1 - ks0);
      constexpr int DT = Cfg::DT;
      constexpr bool SPLIT_TOKENS = Cfg::SPLIT_TOKENS;
      const int tok0 = SPLIT_TOKENS ? 32 * e : 0;  // first token (inside the tile) of this thread's sums
      float psum[DT];
#pragma unroll
      for (int m = 0; m < DT; ++m) psum[m] = 0.f;
      for (uint32_t i = SPLIT_TOKENS ? i_seg0 : i_seg0 + ((i_seg0 ^ (uint32_t)e) & 1u); i < i_end; i += SPLIT_TOKENS ? 1 : 2) {
        float s0 = 1.0f, s1 = 1.0f;
        if (scaled) {
          const uint32_t ss = i % SS;
          w4g_wait<W4G_SC_FULL, ST_TIMEOUT_EPILOGUE>(bar0 + 8 * ss, (i / SS) & 1u, ctl, fail);
          uint16_t h0, h1;
          asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h0) : "r"(sc_addr0 + ss * W4G_SC_BYTES));
          asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h1) : "r"(sc_addr0 + ss * W4G_SC_BYTES + sc_row1));
          s0 = __half2float(__ushort_as_half(h0));
          s1 = __half2float(__ushort_as_half(h1));
          __syncwarp();
          if (lead) w4g_arrive<W4G_SC_EMPTY>(bar0 + 8 * ss);
        }
        const uint32_t slot = i % NSLOT;
        const uint32_t bs = bar0 + 8 * slot;
        w4g_wait<W4G_ACC_FULL, ST_TIMEOUT_EPILOGUE>(bs, (i / NSLOT) & 1u, ctl, fail);
        tc_fence_after_sync();
        const uint32_t ta = tmem_base + lane_addr + slot * (2 * MT) + tok0;
        if constexpr (MT == 16) {
          uint32_t r[32];  // columns 0..15: first half's accumulator, 16..31: second half's
          tmem_ld_32x32b_x32(ta, r);
          tmem_ld_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lead) w4g_arrive<W4G_ACC_EMPTY>(bs);
#pragma unroll
          for (int m = 0; m < 16; m += 2) {
            w4g_fma2(psum[m], psum[m + 1], r[m], r[m + 1], s0);
            w4g_fma2(psum[m], psum[m + 1], r[16 + m], r[17 + m], s1);
          }
        } else {
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {  // 16 columns at a time: half c4 / 2, this thread's tokens 16 * (c4 % 2) ..
            uint32_t r[16];
            tmem_ld_32x32b_x16(ta + (c4 >> 1) * MT + 16 * (c4 & 1), r);
            tmem_ld_wait();
            if (c4 == 3) {
              tc_fence_before_sync();
              __syncwarp();
              if (lead) w4g_arrive<W4G_ACC_EMPTY>(bs);
            }
            const float s = (c4 >> 1) ? s1 : s0;
#pragma unroll
            if constexpr (MT == 64) {  // the paired form costs this tile registers it does not have (spills)
              for (int m = 0; m < 16; ++m) psum[16 * (c4 & 1) + m] = fmaf(__uint_as_float(r[m]), s, psum[16 * (c4 & 1) + m]);
            } else {
              for (int m = 0; m < 16; m += 2)
                w4g_fma2(psum[16 * (c4 & 1) + m], psum[16 * (c4 & 1) + m + 1], r[m], r[m + 1], s);
            }
          }
        }
      }
      i_seg0 = i_end;
      fail = __any_sync(0xffffffffu, fail != 0) ? 1u : 0u;
      // Segment end.  With slab-alternating sets, set 1 hands over its sums (set 0 has read them before it reaches
      // the second barrier below, which set 1 passes before its next hand-over) and set 0 adds them and writes the
      // tile or its split-K partial; with token-split sets each set writes its own tokens.
      const int par = seg_idx & 1;
      ++seg_idx;
      float* xb = xbuf + nl;
      if (!SPLIT_TOKENS && e == 1) {
#pragma unroll
        for (int j = 0; j < DT; ++j) xb[j * W4_BN] = psum[j];
      }
      w4g_epi_bar();
      if constexpr (SMALL) {
        // One segment per CTA.  Set 0 holds the CTA's sums; CTAs 1 .. C-1 of the cluster write theirs into the first
        // CTA's landing area (the raw ring's stages 4 .. 7, never filled in this form) and signal it; the first CTA
        // adds them in rank order and writes the tile.
        if (e == 0) {
#pragma unroll
          for (int j = 0; j < DT; ++j) psum[j] += xb[j * W4_BN];
        }
        float* landing = reinterpret_cast<float*>(raw_base + W4G_SMALL_MAX_SLABS * W4_RAW_PACKED);  // [rank - 1][token][row]
        if (crank != 0) {
          if (e == 0 && !fail) {
            const uint32_t dst = mapa_u32(smem_u32(landing + (size_t)(crank - 1) * (MT * W4_BN) + nl), 0);
#pragma unroll
            for (int j = 0; j < DT; ++j)
              asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(dst + (uint32_t)(j * W4_BN * 4)), "f"(psum[j]) : "memory");
            fence_acq_rel_cluster();
          }
          w4g_epi_bar();  // every thread's stores are issued and fenced before the one signal
          // (test hook, value 2: the last cluster's CTA 1 keeps its signal back, so that the first CTA's wait runs out)
          const bool withheld = dbg.withhold_last_commit == 2 && crank == 1 && cta / csize == G / csize - 1;
          if (warp == W4G_FIRST_EPI_WARP && lane == 0 && !fail && ctl_words[0] == 0 && !withheld)
            mbar_arrive_cluster(mapa_u32(bar0 + W4G_PART_FULL, 0));
        } else {
          bool got = true;
          if (csize > 1) {
            if (lane == 0) {
              const uint64_t t0 = global_timer_ns();
              while (!mbar_try_wait_cluster(reinterpret_cast<uint64_t*>(bar_block + W4G_PART_FULL), 0)) {
                if (ctl_words[0] != 0 || global_timer_ns() - t0 > p.wait_limit_ns) {
                  if (ctl_words[0] == 0) ctl_words[0] = ST_TIMEOUT_EPILOGUE;
                  got = false;
                  break;
                }
              }
            }
            got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
            fence_acq_rel_cluster();
          }
          if (got && e == 0 && !fail && n < p.N) {
            for (int c = 1; c < csize; ++c) {
              const float* src = landing + (size_t)(c - 1) * (MT * W4_BN) + nl;
#pragma unroll
              for (int j = 0; j < DT; ++j) psum[j] += src[j * W4_BN];
            }
#pragma unroll
            for (int j = 0; j < DT; ++j) {
              const int m = m0 + j;
              if (m < p.M) w4_store_out<OUT_BF16, GATHER>(p, Cout, m, n, psum[j]);
            }
          }
        }
        break;
      }
      const long long first_item = (long long)tile * p.KS;
      int b_first = 0, b_last = 0;
      if (!full_tile) {
        b_first = w4_owner(T, G, first_item);
        b_last = w4_owner(T, G, first_item + p.KS - 1);
      }
      if ((SPLIT_TOKENS || e == 0) && !fail) {
        if (!SPLIT_TOKENS) {
#pragma unroll
          for (int j = 0; j < DT; ++j) psum[j] += xb[j * W4_BN];
        }
        if (full_tile) {
          if (n < p.N) {
#pragma unroll
            for (int j = 0; j < DT; ++j) {
              const int m = m0 + tok0 + j;
              if (m < p.M) w4_store_out<OUT_BF16, GATHER>(p, Cout, m, n, psum[j]);
            }
          }
        } else {
          float* dst = p.ws_partials + (size_t)my_slot * (MT * W4_BN) + (size_t)tok0 * W4_BN + nl;
#pragma unroll
          for (int j = 0; j < DT; ++j) dst[j * W4_BN] = psum[j];
          __threadfence();
        }
      }
      // The eight drain warps decide together whether to go on: one thread reads the abort word once and
      // publishes it (with the split-K outcome) in a control word that alternates between two slots, so a fast
      // warp's next write cannot overtake a slow warp's read.
      w4g_epi_bar();
      if (warp == W4G_FIRST_EPI_WARP && lane == 0) {
        uint32_t ctrl = (ctl_words[0] || fail) ? 1u : 0u;
        if (!ctrl && !full_tile) {
          // split tile: count arrivals; the last contributor adds all partials in a fixed order
          const uint32_t old = atomicAdd(p.ws_counters + b_first, 1u);
          if (old == (uint32_t)(b_last - b_first)) ctrl |= 2u;
        }
        epi_ctrl[par] = ctrl;
      }
      w4g_epi_bar();
      const uint32_t ctrl = epi_ctrl[par];
      if (ctrl & 1u) break;
      const bool is_last = (ctrl & 2u) != 0;
      if (is_last && (Cfg::SPLIT_TOKENS || e == 0)) {
        __threadfence();
        if (n < p.N) {
          const int rows = min(Cfg::SPLIT_TOKENS ? 32 * e + 32 : MT, p.M - m0);
#pragma unroll 1
          for (int mb = Cfg::SPLIT_TOKENS ? 32 * e : 0; mb < rows; mb += 16) {
            float sum[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) sum[u] = 0.0f;
#pragma unroll 1
            for (int c = b_first; c <= b_last; ++c) {  // fixed order: results do not depend on arrival order
              const long long c_end = w4_range_begin(T, G, c + 1);
              const int pslot = (c_end >= first_item + p.KS) ? 2 * c : 2 * c + 1;
              const float* src = p.ws_partials + (size_t)pslot * (MT * W4_BN) + (size_t)mb * W4_BN + nl;
              float v[16];
#pragma unroll
              for (int u = 0; u < 16; ++u) v[u] = (mb + u < rows) ? __ldcg(src + u * W4_BN) : 0.0f;
#pragma unroll
              for (int u = 0; u < 16; ++u) sum[u] += v[u];
            }
#pragma unroll
            for (int u = 0; u < 16; ++u) {
              if (mb + u < rows)
                w4_store_out<OUT_BF16, GATHER>(p, Cout, m0 + mb + u, n, sum[u]);
            }
          }
        }
      }
    }
  } else if (warp >= W4G_FIRST_DQ_WARP && warp < W4G_FIRST_MMA_WARP) {
    // ------------------------------------------------------------------ dequant
    // Two sets of eight warps take alternate slabs: set g = wd / 8 converts slabs g, g + 2, ...  Inside a set,
    // warp (q, hf) owns TMEM lanes 32 q .. 32 q + 31 (the quadrant it may touch) and the 128-k half hf of the
    // slab = the packed 16-byte chunks 4 hf .. 4 hf + 3 of a row = the 64 columns of weight stage 2 g + hf.
    // Iteration n = 4 * c + u of a set handles slab 2 n + g: raw stage 2 u + g (its c-th fill, parity c & 1),
    // weight stage 2 g + hf (its n-th use, parity n & 1 = u & 1).
    const int wd = warp - W4G_FIRST_DQ_WARP;
    const int g = wd >> 3;
    const int q = warp & 3;
    const int hf = (wd >> 2) & 1;
    const int row = q * 32 + lane;
    const int sw = row & 7;
    const uint32_t rawr = smem_u32(raw_base) + g * W4_RAW_PACKED + row * 128;  // this thread's row in raw stage g
    // quarter-warps read 8 rows x 8 distinct chunks (128-byte swizzle)
    const uint32_t ch0 = rawr + (((4 * hf + 0) ^ sw) << 4), ch1 = rawr + (((4 * hf + 1) ^ sw) << 4);
    const uint32_t ch2 = rawr + (((4 * hf + 2) ^ sw) << 4), ch3 = rawr + (((4 * hf + 3) ^ sw) << 4);
    const uint32_t zero = (uint32_t)p.zero;
    const uint32_t sub_lo_c = (0x6400u + zero) * 0x00010001u;                     // (1024 + zero) x2
    const uint32_t sub_hi_c = ((0x5400u + (zero << 4)) | 0x8000u) * 0x00010001u;  // -(64 + zero) x2
    // this row's zero point of the half: stage g of the zero ring, second row for the second half of 128-wide groups
    const uint32_t z_addr = smem_u32(z_base) + g * W4G_SC_BYTES + 2 * row + ((p.scale_rows == 2 && hf) ? 256u : 0u);
    const uint32_t st_addr = tmem_w + ((uint32_t)(q * 32) << 16) + (2 * g + hf) * W4G_HALF_COLS;
    const uint32_t bg = bar0 + 8 * g;             // raw stages g, g + 2, g + 4, g + 6
    const uint32_t bws = bar0 + 8 * (2 * g + hf);  // weight stage 2 g + hf
    const bool lead = lane == 0;
    const int n_mine = (n_slabs - g + 1) >> 1;  // slabs g, g + 2, ... below n_slabs
    uint32_t fail = 0;
    for (int nb = 0; nb < n_mine; nb += 4) {
      const uint32_t rphase = (uint32_t)(nb >> 2) & 1u;
      auto step = [&](auto u_) {
        constexpr int u = decltype(u_)::value;
        if (nb + u >= n_mine) return;
        w4g_wait<W4G_RAW_FULL + 16 * u, ST_TIMEOUT_DEQUANT>(bg, rphase, ctl, fail);
        uint32_t sub_lo = sub_lo_c, sub_hi = sub_hi_c;
        if constexpr (ZT) {
          // integer zero z as f16: 1024 + z and 64 + z are exact f16 sums
          uint16_t zh;
          asm volatile("ld.shared.u16 %0, [%1+%2];" : "=h"(zh) : "r"(z_addr), "n"(2 * u * W4G_SC_BYTES));
          uint32_t z2;
          asm("mov.b32 %0, {%1, %1};" : "=r"(z2) : "h"(zh));
          asm("add.rn.f16x2 %0, %1, %2;" : "=r"(sub_lo) : "r"(0x64006400u), "r"(z2));
          asm("add.rn.f16x2 %0, %1, %2;" : "=r"(sub_hi) : "r"(0x54005400u), "r"(z2));
          sub_hi ^= 0x80008000u;
        }
        const uint4 v0 = w4g_lds128<2 * u * W4_RAW_PACKED>(ch0);
        const uint4 v1 = w4g_lds128<2 * u * W4_RAW_PACKED>(ch1);
        const uint4 v2 = w4g_lds128<2 * u * W4_RAW_PACKED>(ch2);
        const uint4 v3 = w4g_lds128<2 * u * W4_RAW_PACKED>(ch3);
        // four batches of 32 weights (16 columns) each, so that few registers are live at a time
        uint32_t o[16];
        w4_dequant8(v0.x, sub_lo, sub_hi, 0u, false, o + 0);
        w4_dequant8(v0.y, sub_lo, sub_hi, 0u, false, o + 4);
        w4_dequant8(v0.z, sub_lo, sub_hi, 0u, false, o + 8);
        w4_dequant8(v0.w, sub_lo, sub_hi, 0u, false, o + 12);
        w4g_wait<W4G_W_EMPTY, ST_TIMEOUT_DEQUANT>(bws, (uint32_t)((u & 1) ^ 1), ctl, fail);
        tc_fence_after_sync();
        tmem_st_32x32b_x16(st_addr, o);
        uint32_t o1[16];
        w4_dequant8(v1.x, sub_lo, sub_hi, 0u, false, o1 + 0);
        w4_dequant8(v1.y, sub_lo, sub_hi, 0u, false, o1 + 4);
        w4_dequant8(v1.z, sub_lo, sub_hi, 0u, false, o1 + 8);
        w4_dequant8(v1.w, sub_lo, sub_hi, 0u, false, o1 + 12);
        tmem_st_32x32b_x16(st_addr + 16, o1);
        uint32_t o2[16];
        w4_dequant8(v2.x, sub_lo, sub_hi, 0u, false, o2 + 0);
        w4_dequant8(v2.y, sub_lo, sub_hi, 0u, false, o2 + 4);
        w4_dequant8(v2.z, sub_lo, sub_hi, 0u, false, o2 + 8);
        w4_dequant8(v2.w, sub_lo, sub_hi, 0u, false, o2 + 12);
        tmem_st_32x32b_x16(st_addr + 32, o2);
        uint32_t o3[16];
        w4_dequant8(v3.x, sub_lo, sub_hi, 0u, false, o3 + 0);
        // the last of the four loads has delivered: the packed bytes are in registers, hand the raw stage back
        __syncwarp();
        if (lead) w4g_arrive<W4G_RAW_EMPTY + 16 * u>(bg);
        w4_dequant8(v3.y, sub_lo, sub_hi, 0u, false, o3 + 4);
        w4_dequant8(v3.z, sub_lo, sub_hi, 0u, false, o3 + 8);
        w4_dequant8(v3.w, sub_lo, sub_hi, 0u, false, o3 + 12);
        tmem_st_32x32b_x16(st_addr + 48, o3);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lead) w4g_arrive<W4G_W_FULL>(bws);
      };
      step(std::integral_constant<int, 0>{});
      step(std::integral_constant<int, 1>{});
      step(std::integral_constant<int, 2>{});
      step(std::integral_constant<int, 3>{});
      fail = __any_sync(0xffffffffu, fail != 0) ? 1u : 0u;
      if (fail) break;
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (SMALL) cluster_sync_all();  // no CTA of the cluster leaves while another may still reach into it
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    if (lane == 0 && ctl_words[0] != 0 && p.status != nullptr) atomicMax(p.status, ctl_words[0]);
  }
}

}  // namespace qg
