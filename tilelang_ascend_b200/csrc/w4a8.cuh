// Fused W4A8 GEMM for sm_100a: C[m,n] = sum_k int32(A[m,k]) * int32(unpack(qB)[n,k]), exact, for up to 128 tokens.
//
// The int4 weights go from HBM to the tensor core without an int8 copy in global memory: the reference
// (examples/dequantize_gemm/example_dequant_gemm_w4a8.py:69-119) and the two-kernel path of this library
// unpack into an [N, K] int8 workspace first, 0.5 + 1 + 1 bytes of traffic per weight instead of 0.5.
// Same pipeline as the W4A16 kernel in w4a16.cuh (TMA ring of packed slabs -> unpack warps -> tcgen05.st into a
// ring of TMEM columns -> tcgen05.mma with the A operand from TMEM -> stream-K epilogue), with kind::i8 MMAs
// (32 k per instruction), int32 accumulators and partial sums, and a three-instruction unpack per eight
// weights, which leaves the kernel bound by the weight stream.
#pragma once

#include "act_quant.cuh"
#include "common.cuh"
#include "w4a16.cuh"

namespace qg {

struct W4A8Params {
  int* C;                // [M, N] int32
  int* ws_partials;      // scratch: 2 * grid slots of [MT][128] int32
  uint32_t* ws_counters; // scratch: grid counters, zeroed by the pre-pass kernel of every call
  const int* row_sums;   // [M] sum_k A[m,k] (signed nibbles only)
  int M, N, K;
  int n_tiles;           // 128-row weight tiles; one token tile (M <= MT)
  int KS;                // 256-wide K slabs per tile
  long long total_items;
  uint32_t* status;
  unsigned long long wait_limit_ns;
};
constexpr int W4I8_W_COLS = W4_SLAB_K / 4;  // TMEM columns per slab of int8 weights (4 per 32-bit column)

template <int MT>
struct W4I8Cfg {
  static constexpr int RAW_STAGES = 8;                 // even, like W_STAGES: a stage always belongs to one warp set
  static constexpr int A_STAGES = (MT <= 32) ? 8 : (MT == 64 ? 4 : 3);
  static constexpr int MMAW = (MT <= 32) ? 4 : (MT == 64 ? 2 : 1);
  static constexpr int W_STAGES = 4;
  static constexpr int A_KB_BYTES = MT * 128;          // one 128-wide K block of int8 activations
  static constexpr int A_BYTES = 2 * A_KB_BYTES;       // one 256-wide slab
  static constexpr int ACC_COLS = 2 * MMAW * MT;
  static constexpr int TMEM_COLS = 512;
  static constexpr int BAR_BYTES = 512;
  static constexpr int SMEM_BYTES = RAW_STAGES * W4_RAW_PACKED + A_STAGES * A_BYTES + BAR_BYTES + 1024;
  static constexpr int CH = (MT < 32) ? 16 : 32;
  static_assert(ACC_COLS + W_STAGES * W4I8_W_COLS <= 512, "tensor memory budget");
  // an MMA issuer takes every MMAW-th slab: with ring depths that are multiples of MMAW it always meets the same
  // stages and every one of their phases, which is what makes its parity waits safe
  static_assert(W_STAGES % MMAW == 0 && A_STAGES % MMAW == 0, "ring depths must be multiples of the issuer count");
};

// Pre-pass: int8 activations [M, K] -> the same values with every group of eight k reordered to
// 0,2,4,6,1,3,5,7 (the byte order the unpack produces), and the row sums.  One block per row.
__global__ void __launch_bounds__(256)
w4a8_prepare_activations(const uint2* __restrict__ in, uint2* __restrict__ out, int* __restrict__ row_sums,
                         uint32_t* __restrict__ counters, int n_counters, int K) {
  __shared__ int red[8];
  pdl_launch_dependents();
  pdl_wait();  // behind another call of this operator: that call's kernel still reads the scratch until it is done
  // the caller's scratch holds anything: the arrival counters start at zero
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_counters; i += gridDim.x * blockDim.x) counters[i] = 0u;
  const int m = blockIdx.x;
  const uint2* src = in + (size_t)m * (K / 8);
  uint2* dst = out + (size_t)m * (K / 8);
  int acc = 0;
  for (int i = threadIdx.x; i < K / 8; i += blockDim.x) {
    const uint2 v = src[i];
    acc = __dp4a((int)v.x, 0x01010101, acc);
    acc = __dp4a((int)v.y, 0x01010101, acc);
    dst[i] = make_uint2(__byte_perm(v.x, v.y, 0x6420), __byte_perm(v.x, v.y, 0x7531));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    int s = 0;
    for (int w = 0; w < 8; ++w) s += red[w];
    row_sums[m] = s;
  }
}

// The same pre-pass with the per-token activation quantiser in front of it, fused: bf16 / f16 activations [M, K] ->
// scale[m] = max(amax, 1e-4) / 127 (optionally rounded up to a power of two), int8 values rint(x / scale) written
// straight in the kernel's byte order, and their row sums.  The arithmetic is act_quant_kernel's (act_quant.cuh),
// so the int8 values and scales are bit-identical to running that kernel first
// (examples/deepseek_v4/act_quant.py:112-142); what disappears is one launch and the int8 round trip through
// memory.  One block per row; a thread keeps up to eight 16-byte chunks of the row in registers between the abs-max
// pass and the quantise pass (K <= 16384), longer rows are read again.
__global__ void __launch_bounds__(256)
w4a8_quant_prepare_activations(const uint4* __restrict__ X, int is_bf16, int round_scale, uint2* __restrict__ out,
                               int* __restrict__ row_sums, float* __restrict__ scales, uint32_t* __restrict__ counters,
                               int n_counters, int K) {
  __shared__ float redf[8];
  __shared__ int red[8];
  pdl_launch_dependents();
  pdl_wait();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_counters; i += gridDim.x * blockDim.x) counters[i] = 0u;
  const int m = blockIdx.x;
  const int chunks = K >> 3;
  const bool bf16 = is_bf16 != 0;
  const uint4* x = X + (size_t)m * chunks;
  uint2* dst = out + (size_t)m * chunks;
  constexpr int KEEP = 8;
  uint4 keep[KEEP];
  uint32_t m2 = 0u;
#pragma unroll
  for (int i = 0; i < KEEP; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c < chunks) {
      keep[i] = __ldg(x + c);
      m2 = aq_absmax8(keep[i], bf16, m2);
    }
  }
  for (int c = threadIdx.x + KEEP * 256; c < chunks; c += 256) m2 = aq_absmax8(__ldg(x + c), bf16, m2);
  float mx = aq_pair_max(m2, bf16);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) redf[threadIdx.x >> 5] = mx;
  __syncthreads();
#pragma unroll
  for (int w = 0; w < 8; ++w) mx = fmaxf(mx, redf[w]);
  const float amax = fmaxf(mx, 1e-4f);
  float scale = __fdiv_rn(amax, 127.0f);
  if (round_scale) scale = aq_pow2_ceil(scale);
  const float rcp = __frcp_rn(scale);
  int acc = 0;
  auto emit = [&](int c, const uint4& v) {
    const uint2 q = aq_quant8(v, bf16, scale, rcp);  // eight int8 values in K order
    acc = __dp4a((int)q.x, 0x01010101, acc);
    acc = __dp4a((int)q.y, 0x01010101, acc);
    dst[c] = make_uint2(__byte_perm(q.x, q.y, 0x6420), __byte_perm(q.x, q.y, 0x7531));
  };
#pragma unroll
  for (int i = 0; i < KEEP; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c < chunks) emit(c, keep[i]);
  }
  for (int c = threadIdx.x + KEEP * 256; c < chunks; c += 256) emit(c, __ldg(x + c));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    int sum = 0;
    for (int w = 0; w < 8; ++w) sum += red[w];
    row_sums[m] = sum;
    scales[m] = scale;
  }
}

template <int MT, bool SIGNED>
__global__ void __launch_bounds__(W4_THREADS, 1)
w4a8_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA,
                 const W4A8Params p) {
  using Cfg = W4I8Cfg<MT>;
  pdl_launch_dependents();  // the next call's pre-pass may become resident; it waits for this grid before it writes
  constexpr int RS = Cfg::RAW_STAGES;
  constexpr int AS = Cfg::A_STAGES;
  constexpr int WS = Cfg::W_STAGES;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* raw_base = smem;
  uint8_t* a_base = smem + RS * W4_RAW_PACKED;
  uint64_t* bars = reinterpret_cast<uint64_t*>(a_base + AS * Cfg::A_BYTES);
  uint64_t* raw_full = bars;
  uint64_t* raw_empty = raw_full + RS;
  uint64_t* a_full = raw_empty + RS;
  uint64_t* a_empty = a_full + AS;
  uint64_t* w_full = a_empty + AS;
  uint64_t* w_empty = w_full + WS;
  uint64_t* tfull = w_empty + WS;
  uint64_t* tempty = tfull + 2;
  uint64_t* drain = tempty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* epi_flag = tmem_slot + 2;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < RS; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], W4_DQ_WARPS / 2);  // the eight warps of the set that takes this slab
    }
    for (int s = 0; s < AS; ++s) {
      mbar_init(&a_full[s], 1);
      mbar_init(&a_empty[s], 1);  // released by the one issuer that took the slab
    }
    for (int s = 0; s < WS; ++s) {
      mbar_init(&w_full[s], W4_DQ_WARPS / 2);
      mbar_init(&w_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], Cfg::MMAW);
      mbar_init(&tempty[i], 4);
    }
    mbar_init(drain, 1);
    *abort_flag = 0;
    epi_flag[0] = epi_flag[1] = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmA);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_w = tmem_base + Cfg::ACC_COLS;  // ring of dequantised-weight columns
  const WaitCtl ctl{abort_flag, p.status, p.wait_limit_ns, 0};

  const int G = gridDim.x;
  const int cta = blockIdx.x;
  const long long T = p.total_items;
  W4SegIter seg{w4_range_begin(T, G, cta), w4_range_begin(T, G, cta + 1), p.KS};
  int tile, ks0, ks1;

  if (warp == 0) {
    // ------------------------------------------- raw producer: packed weights + scales
    if (lane == 0) {
      int rs = 0;
      uint32_t phase = 0, issued_mask = 0, parity_mask = 0;
      bool ok = true;
      const uint32_t tx = W4_RAW_PACKED;
      while (ok && seg.next(tile, ks0, ks1)) {
        const int n0 = tile * W4_BN;
        for (int ks = ks0; ks < ks1; ++ks) {
          if (!mbar_wait(&raw_empty[rs], phase ^ 1u, ctl, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
          uint8_t* dst = raw_base + rs * W4_RAW_PACKED;
          mbar_arrive_expect_tx(&raw_full[rs], tx);
          tma_load_2d(dst, &tmW, &raw_full[rs], ks * (W4_SLAB_K / 2), n0);
          issued_mask |= 1u << rs;
          parity_mask = (parity_mask & ~(1u << rs)) | (phase << rs);
          if (++rs == RS) { rs = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        for (int s = 0; s < RS; ++s) {
          if (!(issued_mask & (1u << s))) continue;
          const uint64_t t0 = global_timer_ns();
          while (!mbar_try_wait(&raw_full[s], (parity_mask >> s) & 1u)) {
            if (global_timer_ns() - t0 > p.wait_limit_ns) {
              if (p.status) atomicMax(p.status, (uint32_t)ST_TIMEOUT_DRAIN);
              break;
            }
          }
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------- activation producer
    if (lane == 0) {
      pdl_wait();  // the reordered activations come from the pre-pass kernel in front of this one
      int as = 0;
      uint32_t phase = 0, issued_mask = 0, parity_mask = 0;
      bool ok = true;
      while (ok && seg.next(tile, ks0, ks1)) {
        for (int ks = ks0; ks < ks1; ++ks) {
          if (!mbar_wait(&a_empty[as], phase ^ 1u, ctl, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
          uint8_t* dstA = a_base + as * Cfg::A_BYTES;
          mbar_arrive_expect_tx(&a_full[as], Cfg::A_BYTES);
#pragma unroll
          for (int kb = 0; kb < 2; ++kb)  // two 128-byte (128 k) blocks of int8 activations per slab
            tma_load_2d(dstA + kb * Cfg::A_KB_BYTES, &tmA, &a_full[as], ks * W4_SLAB_K + kb * 128, 0);
          issued_mask |= 1u << as;
          parity_mask = (parity_mask & ~(1u << as)) | (phase << as);
          if (++as == AS) { as = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        for (int s = 0; s < AS; ++s) {
          if (!(issued_mask & (1u << s))) continue;
          const uint64_t t0 = global_timer_ns();
          while (!mbar_try_wait(&a_full[s], (parity_mask >> s) & 1u)) {
            if (global_timer_ns() - t0 > p.wait_limit_ns) {
              if (p.status) atomicMax(p.status, (uint32_t)ST_TIMEOUT_DRAIN);
              break;
            }
          }
        }
      }
    }
  } else if (warp == 1 || warp >= W4_FIRST_XMMA_WARP) {
    // -------------------------------------------------------------- MMA issuers
    // Issuer w of MMAW takes every MMAW-th slab of this CTA (slab index % MMAW == w), all of its K steps, and
    // accumulates into its own accumulator (columns w*MT of the buffer).  One issuing thread needs about 900
    // cycles per slab for its MMAs, the commits and the barrier round trips, more than the slab's HBM time; with
    // whole slabs dealt round-robin that cost is spread over MMAW threads.
    const int mw = (warp == 1) ? 0 : (warp - W4_FIRST_XMMA_WARP + 1);
    // The issuing warps run converged: all lanes wait, one hardware-elected lane (always the same one) issues - under
    // `if (elect_one_sync())` the compiler keeps the descriptors in uniform registers and the issue cost per MMA drops
    // to about half of what `if (lane == 0)` needs (measured on the f16 kernels).
    if (mw < Cfg::MMAW) {
      constexpr uint32_t idesc = make_idesc(ACC_S32, FMT_S8, FMT_S8, 0, 0, W4_BN, MT);
      const uint64_t desc_hi = make_desc_kmajor(0);  // K-major activation descriptor without its start address
      const uint32_t a_base_u32 = smem_u32(a_base);
      int ws = 0, as = 0;
      uint32_t wphase = 0, aphase = 0;
      int it = 0;
      int turn = 0;  // slab index % MMAW
      bool ok = true;
      while (ok && seg.next(tile, ks0, ks1)) {
        const int buf = it & 1;
        const uint32_t tphase = (it >> 1) & 1;
        if (!mbar_wait_warp(&tempty[buf], tphase ^ 1u, ctl, ST_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d = tmem_base + buf * (Cfg::MMAW * MT) + mw * MT;
        uint32_t started = 0;  // 0 for this issuer's first MMA of the segment: overwrite the accumulator
        for (int ks = ks0; ks < ks1; ++ks) {
          if (turn == mw) {
            if (!mbar_wait_warp(&a_full[as], aphase, ctl, ST_TIMEOUT_MMA)) { ok = false; break; }
            if (!mbar_wait_warp(&w_full[ws], wphase, ctl, ST_TIMEOUT_MMA)) { ok = false; break; }
            tc_fence_after_sync();
            const uint64_t adesc0 = desc_hi | (uint64_t)(((a_base_u32 + as * Cfg::A_BYTES) & 0x3FFFFu) >> 4);
            const uint32_t tW = tmem_w + ws * W4I8_W_COLS;
            if (elect_one_sync()) {
#pragma unroll
              for (int kk = 0; kk < W4_SLAB_K / 32; ++kk) {  // 32 k per MMA: 8 TMEM columns, 32 bytes of smem
                const uint32_t off = (uint32_t)(((kk >> 2) * Cfg::A_KB_BYTES + (kk & 3) * 32) >> 4);
                umma_i8_ts(d, tW + kk * 8, adesc0 + off, idesc, kk == 0 ? started : 1u);
              }
              umma_commit(&w_empty[ws]);
              umma_commit(&a_empty[as]);
            }
            started = 1u;
          }
          if (++turn == Cfg::MMAW) turn = 0;
          if (++ws == WS) { ws = 0; wphase ^= 1u; }
          if (++as == AS) { as = 0; aphase ^= 1u; }
        }
        // the elected lane is the same one every time, so this commit covers the MMAs issued above
        if (ok && elect_one_sync()) umma_commit(&tfull[buf]);
        ++it;
      }
      if (!ok && mw == 0) {
        if (elect_one_sync()) umma_commit(drain);
        if (lane == 0) {
          const uint64_t t0 = global_timer_ns();
          while (!mbar_try_wait(drain, 0)) {
            if (global_timer_ns() - t0 > p.wait_limit_ns) break;
          }
        }
      }
    }
  } else if (warp >= 3 && warp < W4_FIRST_DQ_WARP) {
    // ---------------------------------------------------------------- epilogue
    // int32 accumulators: the MMAW accumulators add exactly; signed nibbles were fed as (value + 8), so
    // 8 * sum_k a[m,k] comes off once, when the tile's full-K sum is written.
    constexpr int CH = Cfg::CH;
    const int q = warp & 3;
    const int nl = q * 32 + lane;  // weight row inside the tile == TMEM lane
    int it = 0, seg_idx = 0;
    long long first_slab = 0;  // CTA-local index of the segment's first slab: issuer (first_slab + i) % MMAW took slab i
    pdl_wait();  // row sums and zeroed counters come from the pre-pass kernel
    while (seg.next(tile, ks0, ks1)) {
      const int buf = it & 1;
      const uint32_t tphase = (it >> 1) & 1;
      ++it;
      const int seg_len = ks1 - ks0;
      const int first_turn = (int)(first_slab % Cfg::MMAW);
      first_slab += seg_len;
      const int n = tile * W4_BN + nl;
      const bool full_tile = (ks0 == 0 && ks1 == p.KS);
      const int my_slot = (ks1 < p.KS) ? 2 * cta + 1 : 2 * cta;
      const bool ok = mbar_wait_warp(&tfull[buf], tphase, ctl, ST_TIMEOUT_EPILOGUE);
      if (ok) {
        tc_fence_after_sync();
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * (Cfg::MMAW * MT);
#pragma unroll 1
        for (int c = 0; c < MT / CH; ++c) {
          uint32_t r[CH];
#pragma unroll
          for (int j = 0; j < CH; ++j) r[j] = 0u;
#pragma unroll
          for (int a = 0; a < Cfg::MMAW; ++a) {
            // issuer a wrote its accumulator in this segment only if one of the segment's slabs was its turn
            if (((a - first_turn + Cfg::MMAW) % Cfg::MMAW) < seg_len) {
              uint32_t r2[CH];
              if constexpr (CH == 16) tmem_ld_32x32b_x16(taddr + a * MT + c * CH, r2);
              else tmem_ld_32x32b_x32(taddr + a * MT + c * CH, r2);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < CH; ++j) r[j] += r2[j];
            }
          }
          if (full_tile) {
            if (n < p.N) {
#pragma unroll
              for (int j = 0; j < CH; ++j) {
                const int m = c * CH + j;
                if (m < p.M) p.C[(size_t)m * p.N + n] = (int)r[j] - (SIGNED ? 8 * __ldg(p.row_sums + m) : 0);
              }
            }
          } else {
            int* dst = p.ws_partials + (size_t)my_slot * (MT * W4_BN) + (size_t)(c * CH) * W4_BN + nl;
#pragma unroll
            for (int j = 0; j < CH; ++j) dst[j * W4_BN] = (int)r[j];
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[buf]);
      }
      // Segment end.  The four epilogue warps decide together whether to go on (a warp that left alone would
      // leave the others waiting at the named barrier for ever): one thread reads the abort flag once and
      // publishes it, with the split-K outcome, in a control word that alternates between two slots by segment.
      const int par = seg_idx & 1;
      ++seg_idx;
      const long long first_item = (long long)tile * p.KS;
      int b_first = 0, b_last = 0;
      if (!full_tile) {
        b_first = w4_owner(T, G, first_item);
        b_last = w4_owner(T, G, first_item + p.KS - 1);
        __threadfence();
      }
      w4_epi_bar();
      if (warp == 3 && lane == 0) {
        uint32_t ctrl = *abort_flag ? 1u : 0u;
        if (!ctrl && !full_tile) {
          // split tile: count arrivals; the last contributor adds the partials up
          const uint32_t old = atomicAdd(p.ws_counters + b_first, 1u);
          if (old == (uint32_t)(b_last - b_first)) ctrl |= 2u;
        }
        epi_flag[par] = ctrl;
      }
      w4_epi_bar();
      const uint32_t ctrl = epi_flag[par];
      if (ctrl & 1u) break;
      const bool is_last = (ctrl & 2u) != 0;
      if (is_last) {
        __threadfence();
        if (n < p.N) {
          constexpr int RU = 16;
          const int rows = min(MT, p.M);
#pragma unroll 1
          for (int mb = 0; mb < rows; mb += RU) {
            int sum[RU];
#pragma unroll
            for (int u = 0; u < RU; ++u) sum[u] = 0;
#pragma unroll 1
            for (int c = b_first; c <= b_last; ++c) {
              const long long c_end = w4_range_begin(T, G, c + 1);
              const int slot = (c_end >= first_item + p.KS) ? 2 * c : 2 * c + 1;
              const int* src = p.ws_partials + (size_t)slot * (MT * W4_BN) + (size_t)mb * W4_BN + nl;
              int v[RU];
#pragma unroll
              for (int u = 0; u < RU; ++u) v[u] = (mb + u < rows) ? __ldcg(src + u * W4_BN) : 0;
#pragma unroll
              for (int u = 0; u < RU; ++u) sum[u] += v[u];
            }
#pragma unroll
            for (int u = 0; u < RU; ++u) {
              if (mb + u < rows)
                p.C[(size_t)(mb + u) * p.N + n] = sum[u] - (SIGNED ? 8 * __ldg(p.row_sums + mb + u) : 0);
            }
          }
        }
      }
    }
  } else if (warp >= W4_FIRST_DQ_WARP && warp < W4_FIRST_XMMA_WARP) {
    // ----------------------------------------------------------------- unpack
    // Two sets of eight warps take alternate slabs, so that a warp's own chain of barrier round trips, shared
    // memory loads and tensor-memory store (about 600 cycles) spans two slab periods instead of one: with
    // every warp on every slab that chain, not the weight stream, set the pace.
    // Warp (set, q, h): slabs with (index & 1) == set, TMEM lanes 32q..32q+31, K half h of the slab = packed
    // 16-byte chunks 4h..4h+3 of the row = 128 int8 = 32 TMEM columns.  Word x holds nibbles n0..n7 of eight
    // consecutive k: (x & 0x0f0f0f0f) = bytes (n0, n2, n4, n6), ((x >> 4) & 0x0f0f0f0f) = (n1, n3, n5, n7); the
    // pre-pass stores the activations in that same order, so no byte shuffle is needed.  Two's-complement
    // nibbles are biased by XOR 8 (value + 8 in 0..15) in the same lop3.
    const int wd = warp - W4_FIRST_DQ_WARP;
    const int q = warp & 3;
    const int h = (wd >> 2) & 1;
    const int set = wd >> 3;
    const int row = q * 32 + lane;
    const int sw = row & 7;
    uint32_t off[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) off[c] = row * 128 + (((4 * h + c) ^ sw) << 4);
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const long long n_slabs = seg.end - seg.item;  // slabs of this CTA, in order
    bool ok = true;
    for (long long i = set; ok && i < n_slabs; i += 2) {
      const int rs = (int)(i % RS), ws = (int)(i % WS);
      const uint32_t rphase = (uint32_t)((i / RS) & 1), wphase = (uint32_t)((i / WS) & 1);
      if (!mbar_wait_warp(&raw_full[rs], rphase, ctl, ST_TIMEOUT_DEQUANT)) { ok = false; break; }
      const uint8_t* rawp = raw_base + rs * W4_RAW_PACKED;
      uint32_t o[32];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint4 v = *reinterpret_cast<const uint4*>(rawp + off[c]);
        const uint32_t x[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const uint32_t y = x[e] >> 4;
          if (SIGNED) {
            asm("lop3.b32 %0, %1, 0x0f0f0f0f, 0x08080808, 0x6a;" : "=r"(o[8 * c + 2 * e]) : "r"(x[e]));
            asm("lop3.b32 %0, %1, 0x0f0f0f0f, 0x08080808, 0x6a;" : "=r"(o[8 * c + 2 * e + 1]) : "r"(y));
          } else {
            o[8 * c + 2 * e] = x[e] & 0x0f0f0f0fu;
            o[8 * c + 2 * e + 1] = y & 0x0f0f0f0fu;
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&raw_empty[rs]);

      if (!mbar_wait_warp(&w_empty[ws], wphase ^ 1u, ctl, ST_TIMEOUT_DEQUANT)) { ok = false; break; }
      tc_fence_after_sync();
      tmem_st_32x32b_x32(tmem_w + lane_addr + ws * W4I8_W_COLS + h * 32, o);
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&w_full[ws]);
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace qg
