// W8A8 quantized (batched) matmul for sm_100a:
//   C[b, m, n] = cast( float(sum_k int32(A[b,m,k]) * int32(B[b,k,n])) [* scale_a[m]] * scale_b[n] )
//
// Persistent, warp-specialised kernel. One CTA per SM walks a list of 128 x BN output tiles:
//   warp 0      TMA producer: A tile [128 x 128 B] and B tile into a multistage shared-memory ring
//   warp 1      tcgen05.mma kind::i8 issuer; int32 accumulators live in tensor memory, double buffered
//   warps 2..5  epilogue: tcgen05.ld -> cvt.rn.f32.s32 -> fp32 scale(s) -> cvt.rn f16/bf16 -> 16-byte stores
// B is consumed in the operator's own [K, N] row-major layout as an MN-major operand (no transpose
// pass), or in [N, K] layout as a K-major operand.
#pragma once

#include "common.cuh"

namespace qg {

struct W8A8Params {
  const float* scale_b;
  const float* scale_a;  // nullable
  void* C;               // [batch, M, N] f16 / bf16
  int32_t* acc_out;      // nullable: raw int32 accumulators [batch, M, N]
  int batch, M, N, K;
  int sb_mode;  // 0: one value for all; 1: [N]; 2: [batch, N]
  int sa_mode;  // 0: none; 1: [M]; 2: [batch, M]
  int m_tiles, n_tiles, num_tiles, k_blocks;
  int group_m;  // tile rasterisation: the tiles of `group_m` row blocks are walked column block by column block

  int bn;            // columns per tile actually computed: a multiple of 32, at most the kernel's BN
  uint32_t* status;  // nullable device word
  unsigned long long wait_limit_ns;
  // Grouped (ragged) form: A and C are [M, K] / [M, N] stacks of row groups, B is [groups, ...]; row block i
  // of the table is (group, first row, valid rows <= 128).  Null for the plain and batched forms.
  const int* meta;
  int groups;
  // Tail split: work items from `split_from` on are half-width tiles (item split_from + 2i + h is the left or
  // right half of tile split_from + i), so that the last, partly filled round of the persistent grid keeps
  // twice as many SMs busy for about half as long.  num_items = num_tiles when nothing is split.
  int split_from, num_items;
  int tma_store;  // C is written with tiled bulk stores from a shared-memory staging tile (needs bn % 64 == 0)
  // Gathered form: n_dst > 0 destinations (tensor maps in the kernel's W8Dst argument, one [M, ldc] buffer per
  // rank) receive every tile at column col0 + n instead of the single C.
  int n_dst, col0;
};

// Output tensor maps of the gathered form (unused entries are copies of the first).
struct W8Dst {
  CUtensorMap m[8];
};

// One output tile's coordinates: batch index of B / scale_b, batch index of A / C / scale_a, first row, valid rows.
struct W8Tile {
  int bB, bA, m0, rows, n0, bn;  // n0: first column, bn: columns of this item
};

constexpr int W8_BM = 128;      // tile rows (= MMA M, one TMEM lane per row)
constexpr int W8_BK = 128;      // K bytes per pipeline stage (one 128-byte swizzle atom)
constexpr int W8_UMMA_K = 32;   // K per tcgen05.mma for 8-bit operands
constexpr int W8_THREADS = 192;

template <int BN>
struct W8Cfg {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int A_BYTES = W8_BM * W8_BK;
  static constexpr int B_BYTES = BN * W8_BK;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int BAR_BYTES = 256;
  static constexpr int SCALE_BYTES = 4 * BN * 4;  // each epilogue warp's copy of the tile's column scales
  static constexpr int OUT_BYTES = 4 * 4096;      // each epilogue warp's staging tile: 32 rows x 64 outputs
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + OUT_BYTES + BAR_BYTES + SCALE_BYTES + 1024;  // + alignment slack
};

__device__ __forceinline__ void w8_decode_tile(const W8A8Params& p, int tile, int& b, int& m_blk, int& n_blk) {
  const int per_batch = p.m_tiles * p.n_tiles;
  b = tile / per_batch;
  const int r = tile - b * per_batch;
  const int band = p.group_m * p.n_tiles;
  const int g = r / band;
  const int first_m = g * p.group_m;
  const int gsz = min(p.m_tiles - first_m, p.group_m);
  const int in_band = r - g * band;
  m_blk = first_m + in_band % gsz;
  n_blk = in_band / gsz;
}

__device__ __forceinline__ W8Tile w8_tile(const W8A8Params& p, int item) {
  int b, m_blk, n_blk;
  W8Tile t;
  if (item < p.split_from) {
    w8_decode_tile(p, item, b, m_blk, n_blk);
    t.n0 = n_blk * p.bn;
    t.bn = p.bn;
  } else {
    const int h = item - p.split_from;
    w8_decode_tile(p, p.split_from + (h >> 1), b, m_blk, n_blk);
    t.bn = p.bn >> 1;
    t.n0 = n_blk * p.bn + (h & 1) * t.bn;
  }
  if (p.meta == nullptr) {
    t.bB = t.bA = b;
    t.m0 = m_blk * W8_BM;
    t.rows = min(W8_BM, p.M - t.m0);
  } else {
    t.bB = __ldg(p.meta + 3 * m_blk);
    t.bA = 0;
    t.m0 = __ldg(p.meta + 3 * m_blk + 1);
    t.rows = min(__ldg(p.meta + 3 * m_blk + 2), W8_BM);
    // a table entry that points outside the tensors computes nothing (loads are bounds-checked by TMA)
    if (t.bB < 0 || t.bB >= p.groups || t.m0 < 0 || t.m0 >= p.M) { t.bB = 0; t.m0 = 0; t.rows = 0; }
    t.rows = min(t.rows, p.M - t.m0);
  }
  return t;
}

// F16 = true runs the same pipeline on f16 operands (kind::f16, fp32 accumulators, no scales): one MMA K step
// is 32 bytes for both element types, so with K counted in bytes (p.K, p.k_blocks) nothing else changes.  It
// serves the large-token W4A16 path, whose weights are dequantised to f16 once and then multiplied here.
//
// SPLITK = true is the form for grids that would leave more than half of the SMs idle (fewer 128 x 256 tiles than
// half the SM count): the kernel is launched in clusters of two CTAs, one tile per cluster; each CTA accumulates
// one half of the K range in its own tensor memory; then each CTA writes its int32 accumulators of the OTHER CTA's
// half of the columns into that CTA's shared memory (the pipeline stages, idle by then) through distributed shared
// memory, adds what it received to its own half and runs the epilogue for that half - an exact integer sum, so the
// result is bit-identical to the unsplit kernel's, the exchange runs in both directions at once and each CTA
// converts and stores half a tile.  The counterpart in the
// reference is the K split of examples/gemm_splitk/example_tilelang_gemm_splitk.py:15-48, whose partial tiles meet
// in global memory through atomic adds (src/tl_templates/ascend/common.h:249-259).
template <int BN, bool B_NK, bool OUT_BF16, bool F16 = false, bool SPLITK = false>
__global__ void __launch_bounds__(W8_THREADS, 1)
w8a8_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ W8Dst tmCs, const W8A8Params p) {
  using Cfg = W8Cfg<BN>;
  static_assert(!(SPLITK && F16), "the split form adds int32 partial sums");
  const CUtensorMap& tmC = tmCs.m[0];
  constexpr int STAGES = Cfg::STAGES;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* out_stage = smem + STAGES * Cfg::STAGE_BYTES;  // 1024-byte aligned: 128-byte swizzled staging tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(out_stage + Cfg::OUT_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = tfull + 2;
  uint64_t* drain = tempty + 2;
  uint64_t* stages_free = drain + 1;    // split form: the peer's MMAs have finished reading the peer's stages
  uint64_t* partial_full = drain + 2;   // split form: the peer's accumulators for this CTA's columns have arrived
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain + 3);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // split form: CTA `crank` of the pair takes the k blocks [kb_begin, kb_end) of tile (block index / 2)
  const int crank = SPLITK ? (int)cluster_ctarank() : 0;
  const int tile_first = SPLITK ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int tile_stride = SPLITK ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int kb_begin = SPLITK ? (crank ? p.k_blocks / 2 : 0) : 0;
  const int kb_end = SPLITK ? (crank ? p.k_blocks : p.k_blocks / 2) : p.k_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(stages_free, 4);
    mbar_init(partial_full, 4);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 4);
    }
    if (p.tma_store) tma_prefetch_desc(&tmC);
    mbar_init(drain, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if constexpr (SPLITK) cluster_sync_all();  // both CTAs' barriers exist before either signals the other's
  const uint32_t tmem_base = *tmem_slot;
  const WaitCtl ctl{abort_flag, p.status, p.wait_limit_ns};

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, issued_mask = 0, parity_mask = 0;
      bool ok = true;
      for (int tile = tile_first; ok && tile < p.num_items; tile += tile_stride) {
        const W8Tile t = w8_tile(p, tile);
        const int m0 = t.m0, n0 = t.n0;
        const int b_boxes = B_NK ? 1 : (t.bn + 127) / 128;  // 128-column boxes of B actually needed
        const uint32_t tx = Cfg::A_BYTES + (B_NK ? (uint32_t)Cfg::B_BYTES : (uint32_t)(b_boxes * W8_BK * 128));
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, ctl, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
          uint8_t* sA = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sB = sA + Cfg::A_BYTES;
          mbar_arrive_expect_tx(&full[stage], tx);
          tma_load_3d(sA, &tmA, &full[stage], kb * W8_BK, m0, t.bA);
          if constexpr (B_NK) {
            tma_load_3d(sB, &tmB, &full[stage], kb * W8_BK, n0, t.bB);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 128; ++c)
              if (c < b_boxes) tma_load_3d(sB + c * (W8_BK * 128), &tmB, &full[stage], n0 + c * 128, kb * W8_BK, t.bB);
          }
          issued_mask |= 1u << stage;
          parity_mask = (parity_mask & ~(1u << stage)) | (phase << stage);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // Gave up: wait (bounded) until every bulk copy already issued has landed before the CTA may exit.
        for (int s = 0; s < STAGES; ++s) {
          if (!(issued_mask & (1u << s))) continue;
          const uint64_t t0 = global_timer_ns();
          while (!mbar_try_wait(&full[s], (parity_mask >> s) & 1u)) {
            if (global_timer_ns() - t0 > p.wait_limit_ns) {
              if (p.status) atomicMax(p.status, (uint32_t)ST_TIMEOUT_DRAIN);
              break;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = tile_first; ok && tile < p.num_items; tile += tile_stride, ++it) {
        const uint32_t bn = (uint32_t)((tile < p.split_from) ? p.bn : (p.bn >> 1));
        const uint32_t idesc = F16 ? make_idesc(ACC_F32, FMT_F16, FMT_F16, 0, B_NK ? 0 : 1, W8_BM, bn)
                                   : make_idesc(ACC_S32, FMT_S8, FMT_S8, 0, B_NK ? 0 : 1, W8_BM, bn);
        const int buf = it & 1;
        const uint32_t tphase = (it >> 1) & 1;
        if (!mbar_wait(&tempty[buf], tphase ^ 1u, ctl, ST_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d = tmem_base + buf * BN;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(&full[stage], phase, ctl, ST_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sA = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t sB = sA + Cfg::A_BYTES;
          const uint64_t a0 = make_desc_kmajor(sA);
#pragma unroll
          for (int k = 0; k < W8_BK / W8_UMMA_K; ++k) {
            const uint64_t adesc = a0 + (uint64_t)((k * W8_UMMA_K) >> 4);
            uint64_t bdesc;
            if constexpr (B_NK) {
              bdesc = make_desc_kmajor(sB) + (uint64_t)((k * W8_UMMA_K) >> 4);
            } else {
              // [K rows][128 B of N]: 32 K rows per MMA = 4096 B; the next 128 columns are one box (16 KB) further.
              bdesc = make_desc_mnmajor(sB + k * (W8_UMMA_K * 128), W8_BK * 128);
            }
            if constexpr (F16) umma_f16_ss(d, adesc, bdesc, idesc, ((kb - kb_begin) | k) != 0 ? 1u : 0u);
            else umma_i8_ss(d, adesc, bdesc, idesc, ((kb - kb_begin) | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(&tfull[buf]);
      }
      if (!ok) {
        umma_commit(drain);
        const uint64_t t0 = global_timer_ns();
        while (!mbar_try_wait(drain, 0)) {
          if (global_timer_ns() - t0 > p.wait_limit_ns) break;
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    // Each warp stages the tile's column scales in its own piece of shared memory BEFORE it waits for the
    // accumulators (the loads hide behind the main loop), and keeps the next 32-column chunk's tcgen05.ld in
    // flight while it converts and stores the current one.
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    const uint64_t pol_out = l2_policy_evict_first();  // the output is written once and not read here
    float* sb_s = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + Cfg::BAR_BYTES) + q * BN;
    uint8_t* my_stage = out_stage + q * 4096;  // [32 rows][128 B], 16-byte piece j of row r at (j ^ (r & 7))
    int it = 0;
    // split form: the other CTA's accumulators travel through CTA 0's pipeline stages, one 16-byte piece per
    // (row, four columns): piece (col / 4, row) at ((col / 4) * 128 + row) * 16, so that a warp's 32 rows are
    // 512 contiguous bytes for the sender's stores and the receiver's loads alike
    const uint32_t part_row = smem_u32(smem) + (uint32_t)(q * 32 + lane) * 16u;
    for (int tile = tile_first; tile < p.num_items; tile += tile_stride, ++it) {
      const W8Tile t = w8_tile(p, tile);
      const int buf = it & 1;
      const uint32_t tphase = (it >> 1) & 1;
      const int m = t.m0 + q * 32 + lane;
      const bool row_ok = q * 32 + lane < t.rows;
      float sa = 1.0f;
      if (p.sa_mode != 0 && row_ok) sa = __ldg(p.scale_a + (p.sa_mode == 2 ? (size_t)t.bA * p.M : 0) + m);
      if (!F16 && p.C != nullptr) {
        const float* sbp = p.scale_b + (p.sb_mode == 2 ? (size_t)t.bB * p.N : 0);
        __syncwarp();  // the previous tile's reads of sb_s are done
        for (int c = lane; c < t.bn; c += 32) {
          const int n = t.n0 + c;
          sb_s[c] = (p.sb_mode == 0) ? __ldg(sbp) : (n < p.N ? __ldg(sbp + n) : 0.f);
        }
        __syncwarp();
      }
      if (!mbar_wait_warp(&tfull[buf], tphase, ctl, ST_TIMEOUT_EPILOGUE)) break;
      tc_fence_after_sync();
      // Split form: each CTA of the pair finishes ONE half of the tile's columns (CTA r: columns r * bn/2 ...): it sends
      // its accumulators of the other half into the peer's pipeline stages and receives the peer's for its own, so
      // that the exchange runs in both directions at once and each CTA converts and stores half a tile.
      int c_begin = 0, c_end = t.bn >> 5;
      if constexpr (SPLITK) {
        const uint32_t taddr_s = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
        const uint32_t peer = (uint32_t)(crank ^ 1);
        const int half_chunks = t.bn >> 6;  // 32-column chunks per half
        // this CTA's MMAs are done (tfull): the peer may write into its stages
        if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(stages_free), peer));
        // ... and the peer's are done when its four epilogue warps have said so here
        if (!mbar_wait_warp(stages_free, 0, ctl, ST_TIMEOUT_EPILOGUE)) break;
        const uint32_t dst_row = mapa_u32(part_row, peer);
#pragma unroll 1
        for (int c = 0; c < half_chunks; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr_s + ((int)peer * half_chunks + c) * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int jj = 0; jj < 8; ++jj)
            st_cluster_v4(dst_row + (uint32_t)((c * 8 + jj) * 128 * 16), r[4 * jj], r[4 * jj + 1], r[4 * jj + 2], r[4 * jj + 3]);
        }
        fence_acq_rel_cluster();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(partial_full), peer));
        // the peer's sums for this CTA's half
        bool got = true;
        if (lane == 0) {
          const uint64_t t0 = global_timer_ns();
          while (!mbar_try_wait_cluster(partial_full, 0)) {
            if (*abort_flag || global_timer_ns() - t0 > p.wait_limit_ns) {
              *abort_flag = 1u;
              if (p.status) atomicMax(p.status, (uint32_t)ST_TIMEOUT_EPILOGUE);
              got = false;
              break;
            }
          }
        }
        got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
        if (!got) break;
        fence_acq_rel_cluster();
        c_begin = crank * half_chunks;
        c_end = c_begin + half_chunks;
      }
      const size_t row_off = ((size_t)t.bA * p.M + (row_ok ? m : 0)) * (size_t)p.N;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
      const int chunks = c_end;
      // Whole row blocks go out as tiled bulk stores (coalesced, clipped at the tensor's edge); a partial
      // block of the grouped form must not touch the rows after it and uses per-row stores.
      const bool tma_out = p.tma_store != 0 && (p.meta == nullptr || t.rows == W8_BM);
      uint32_t r[2][32];
      tmem_ld_32x32b_x32(taddr + c_begin * 32, r[0]);
#pragma unroll 1
      for (int c2 = c_begin; c2 < chunks; c2 += 2) {
        if (tma_out) {  // the previous bulk store has read the staging tile
          if (lane == 0) bulk_wait_group_read0();
          __syncwarp();
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int c = c2 + h;
          if (c >= chunks) break;
          tmem_ld_wait();                                                     // chunk c is in r[h]
          if (c + 1 < chunks) tmem_ld_32x32b_x32(taddr + (c + 1) * 32, r[h ^ 1]);  // chunk c + 1 in flight
          if constexpr (SPLITK) {  // add the other CTA's half of the K range (exact: int32)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              uint4 pv;
              asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(pv.x), "=r"(pv.y), "=r"(pv.z), "=r"(pv.w)
                           : "r"(part_row + (uint32_t)(((c - c_begin) * 8 + j) * 128 * 16)));
              r[h][4 * j] += pv.x;
              r[h][4 * j + 1] += pv.y;
              r[h][4 * j + 2] += pv.z;
              r[h][4 * j + 3] += pv.w;
            }
          }
          const int n = t.n0 + c * 32;
          if (row_ok && n < p.N && p.acc_out != nullptr) {
            int4* dst = reinterpret_cast<int4*>(p.acc_out + row_off + n);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (n + 4 * j < p.N)
                dst[j] = make_int4((int)r[h][4 * j], (int)r[h][4 * j + 1], (int)r[h][4 * j + 2], (int)r[h][4 * j + 3]);
          }
          if (tma_out) {
            if (n < p.N) {
              const float4* sv = reinterpret_cast<const float4*>(sb_s + c * 32);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float4 s_lo = sv[2 * j], s_hi = sv[2 * j + 1];
                const float sc[8] = {s_lo.x, s_lo.y, s_lo.z, s_lo.w, s_hi.x, s_hi.y, s_hi.z, s_hi.w};
                uint32_t o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int col = 8 * j + 2 * e;
                  float f0, f1;
                  if constexpr (F16) {
                    f0 = __uint_as_float(r[h][col]);
                    f1 = __uint_as_float(r[h][col + 1]);
                  } else {
                    f0 = __int2float_rn((int)r[h][col]);
                    f1 = __int2float_rn((int)r[h][col + 1]);
                    if (p.sa_mode != 0) { f0 = __fmul_rn(f0, sa); f1 = __fmul_rn(f1, sa); }
                    f0 = __fmul_rn(f0, sc[2 * e]);
                    f1 = __fmul_rn(f1, sc[2 * e + 1]);
                  }
                  o[e] = pack_out2<OUT_BF16>(f0, f1);
                }
                *reinterpret_cast<uint4*>(my_stage + lane * 128 + (((h * 4 + j) ^ (lane & 7)) << 4)) =
                    make_uint4(o[0], o[1], o[2], o[3]);
              }
            }
          } else if (row_ok && n < p.N) {
            if (p.C != nullptr) {
              uint16_t* cbase = reinterpret_cast<uint16_t*>(p.C) + row_off + n;
              const float4* sv = reinterpret_cast<const float4*>(sb_s + c * 32);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (n + 8 * j < p.N) {
                  const float4 s_lo = sv[2 * j], s_hi = sv[2 * j + 1];
                  const float sc[8] = {s_lo.x, s_lo.y, s_lo.z, s_lo.w, s_hi.x, s_hi.y, s_hi.z, s_hi.w};
                  uint32_t o[4];
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const int col = 8 * j + 2 * e;
                    float f0, f1;
                    if constexpr (F16) {
                      f0 = __uint_as_float(r[h][col]);
                      f1 = __uint_as_float(r[h][col + 1]);
                    } else {
                      f0 = __int2float_rn((int)r[h][col]);
                      f1 = __int2float_rn((int)r[h][col + 1]);
                      if (p.sa_mode != 0) { f0 = __fmul_rn(f0, sa); f1 = __fmul_rn(f1, sa); }
                      f0 = __fmul_rn(f0, sc[2 * e]);
                      f1 = __fmul_rn(f1, sc[2 * e + 1]);
                    }
                    o[e] = pack_out2<OUT_BF16>(f0, f1);
                  }
                  *reinterpret_cast<uint4*>(cbase + 8 * j) = make_uint4(o[0], o[1], o[2], o[3]);
                }
              }
            }
          }
        }
        if (tma_out && t.n0 + c2 * 32 < p.N && t.m0 + q * 32 < p.M) {  // a box wholly outside is not issued
          fence_proxy_async_smem();  // this thread's staging writes are visible to the bulk-copy engine
          __syncwarp();
          if (lane == 0) {
            if (p.n_dst == 0) {
              tma_store_3d_hint(&tmC, my_stage, t.n0 + c2 * 32, t.m0 + q * 32, t.bA, pol_out);
            } else {
              for (int d = 0; d < p.n_dst; ++d)
                tma_store_3d_hint(&tmCs.m[d], my_stage, p.col0 + t.n0 + c2 * 32, t.m0 + q * 32, 0, pol_out);
            }
            bulk_commit_group();
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[buf]);
    }
    if (lane == 0) bulk_wait_group_read0();  // the staging tile must outlive the last bulk store's read
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (SPLITK) cluster_sync_all();  // neither CTA of the pair leaves while the other may still reach into it
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace qg
