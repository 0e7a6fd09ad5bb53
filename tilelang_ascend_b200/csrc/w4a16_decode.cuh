// W4A16 decode variant (few tokens, memory bound) for sm_100a.
//
// With at most 16 tokens the GEMM is a weight stream: every packed byte is read once from HBM and used for a
// handful of tokens.  Measured on B200, tcgen05.mma with a 16-token N costs about 94 cycles per K=16 step
// whatever the accumulator layout (fixed tensor-memory operand/accumulator traffic per instruction), i.e.
// 0.8 us per 16 KB of packed weights against 0.37 us of HBM time, so this variant keeps the weights in
// registers all the way: TMA ring -> 4-byte shared-memory loads -> lop3 conversion -> mma.sync.m16n8k16
// with the weights as the register A operand.  The tcgen05 kernel in w4a16.cuh serves larger token counts.
//
//   warp 0        TMA producer: per 256-wide K slab one stage = packed weights [128 rows x 128 B],
//                 the slab's scales, and the prepared activations [MT tokens x 256 k]
//   warps 1..16   compute: warp (rb, kh) owns weight rows 16*rb .. 16*rb+15 and the K half kh of every slab
//   warp 17       finisher: adds the two K halves of a finished segment, writes the tile or runs the split-K
//                 hand-over (partial sum, fence, arrival counter, fixed-order reduction by the last arriver),
//                 so that the compute warps go straight on to the next segment
//
// Numerics: products (q - zero) * a are exact in the tensor core and accumulate in fp32 per quantisation
// group; the group's fp32 sum is then multiplied by the group scale.  With one token set to a unit vector
// this reproduces half(q - zero) * s bit for bit; in general it differs from multiplying each weight by the
// scale in f16 first only by that product's own rounding (2^-11 relative per term).
// The activations come from the same pre-pass as in w4a16.cuh (f16, every group of eight K values in the
// order 0,4,1,5,2,6,3,7), which is exactly the pairing the lop3 conversion produces.
#pragma once

#include "common.cuh"
#include "w4a16.cuh"

namespace qg {

constexpr int W4D_CWARPS = 16;
constexpr int W4D_FIN_WARP = 1 + W4D_CWARPS;        // 17
constexpr int W4D_THREADS = (2 + W4D_CWARPS) * 32;  // 576

template <int NB>  // NB blocks of 8 tokens (one mma.sync N each)
struct W4DCfg {
  static constexpr int MT = 8 * NB;                           // tokens per tile
  static constexpr int A_KB_BYTES = MT * 128;                 // one 64-wide K block of activations
  static constexpr int STAGE_BYTES = W4_RAW_BYTES + 4 * A_KB_BYTES;
  static constexpr int STAGES = (NB == 1) ? 9 : 7;
  static constexpr int RED_TILE = MT * W4_BN;                 // floats of one K half's tile
  static constexpr int RED_BYTES = 2 * 2 * RED_TILE * 4;      // two buffers x two K halves, handed to the finisher
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + RED_BYTES + BAR_BYTES + 1024;
};

// Eight nibbles of x -> (n - zero) as f16 pairs (n0,n4) (n1,n5) (n2,n6) (n3,n7); no scale.
__device__ __forceinline__ void w4d_convert8(uint32_t x, uint32_t sub_lo, uint32_t sub_hi, uint32_t (&h)[4]) {
  uint32_t lo0, hi0, lo1, hi1;
  const uint32_t y = x >> 8;
  asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(lo0) : "r"(x));
  asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(hi0) : "r"(x));
  asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(lo1) : "r"(y));
  asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(hi1) : "r"(y));
  const uint32_t sixteenth = 0x2C002C00u;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(h[0]) : "r"(lo0), "r"(sub_lo));
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(h[1]) : "r"(hi0), "r"(sixteenth), "r"(sub_hi));
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(h[2]) : "r"(lo1), "r"(sub_lo));
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(h[3]) : "r"(hi1), "r"(sixteenth), "r"(sub_hi));
}

// D(16x8, fp32) = A(16x16, f16, row) * B(16x8, f16, col) + C
__device__ __forceinline__ void w4d_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1, const float (&c)[4]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%10, %11, %12, %13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

// Four fp32 results -> four f16 / bf16 outputs, one 8-byte store.
template <bool OUT_BF16>
__device__ __forceinline__ void w4d_store4(uint16_t* dst, const float4& v) {
  uint2 o;
  if (OUT_BF16) {
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
  } else {
    o.x = pack_f16x2(v.x, v.y);
    o.y = pack_f16x2(v.z, v.w);
  }
  *reinterpret_cast<uint2*>(dst) = o;
}

// FLUSH: number of 32-wide K chunks per quantisation group inside a warp's 128-wide K half (4 when the
// group is 128 or larger, 2 for 64, 1 for 32); 0 = no scales (raw nibble values).
template <int FLUSH, int NB, bool OUT_BF16>
__global__ void __launch_bounds__(W4D_THREADS, 1)
w4a16_decode_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmS,
                    const __grid_constant__ CUtensorMap tmA, const W4A16Params p) {
  using Cfg = W4DCfg<NB>;
  pdl_launch_dependents();  // the next call's pre-pass may become resident; it waits for this grid before it writes
  constexpr int MT = Cfg::MT;
  constexpr int ST = Cfg::STAGES;
  constexpr bool SCALED = FLUSH != 0;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* red = reinterpret_cast<float*>(smem + ST * Cfg::STAGE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ST * Cfg::STAGE_BYTES + Cfg::RED_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + ST;
  uint64_t* red_full = empty + ST;   // [2] compute warps -> finisher
  uint64_t* red_empty = red_full + 2;  // [2] finisher -> compute warps
  volatile uint32_t* abort_flag = reinterpret_cast<uint32_t*>(red_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < ST; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], W4D_CWARPS);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&red_full[i], W4D_CWARPS);
      mbar_init(&red_empty[i], 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmA);
    if (SCALED) tma_prefetch_desc(&tmS);
  }
  __syncthreads();
  const WaitCtl ctl{abort_flag, p.status, p.wait_limit_ns, 0};

  const int G = gridDim.x;
  const int cta = blockIdx.x;
  const long long T = p.total_items;
  W4SegIter seg{w4_range_begin(T, G, cta), w4_range_begin(T, G, cta + 1), p.KS};
  int tile, ks0, ks1;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0, issued_mask = 0, parity_mask = 0;
      bool ok = true;
      const uint32_t tx = W4_RAW_PACKED + (SCALED ? p.scale_rows * 256 : 0) + 4 * Cfg::A_KB_BYTES;
      bool waited = false;  // the activations come from the pre-pass kernel in front: wait for it once, after
                            // the first weight loads are on their way
      while (ok && seg.next(tile, ks0, ks1)) {
        int b, n0, m0;
        w4_tile_coords(p, tile, MT, b, n0, m0);
        for (int ks = ks0; ks < ks1; ++ks) {
          if (!mbar_wait(&empty[s], phase ^ 1u, ctl, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
          uint8_t* dst = smem + s * Cfg::STAGE_BYTES;
          mbar_arrive_expect_tx(&full[s], tx);
          tma_load_3d(dst, &tmW, &full[s], ks * (W4_SLAB_K / 2), n0, b);
          if (SCALED) {
            const int srow = (p.group <= W4_SLAB_K) ? ks * p.scale_rows : (ks * W4_SLAB_K) / p.group;
            tma_load_3d(dst + W4_RAW_PACKED, &tmS, &full[s], n0, srow, b);
          }
          if (!waited) { pdl_wait(); waited = true; }
#pragma unroll
          for (int kb = 0; kb < 4; ++kb)
            tma_load_3d(dst + W4_RAW_BYTES + kb * Cfg::A_KB_BYTES, &tmA, &full[s], ks * W4_SLAB_K + kb * 64, m0, b);
          issued_mask |= 1u << s;
          parity_mask = (parity_mask & ~(1u << s)) | (phase << s);
          if (++s == ST) { s = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        for (int i = 0; i < ST; ++i) {
          if (!(issued_mask & (1u << i))) continue;
          const uint64_t t0 = global_timer_ns();
          while (!mbar_try_wait(&full[i], (parity_mask >> i) & 1u)) {
            if (global_timer_ns() - t0 > p.wait_limit_ns) {
              if (p.status) atomicMax(p.status, (uint32_t)ST_TIMEOUT_DRAIN);
              break;
            }
          }
        }
      }
    }
    return;  // the producer warp takes no part in the compute warps' named barrier
  }

  if (warp == W4D_FIN_WARP) {
    // ---------------------------------------------------------------- finisher
    // Lane l owns the float4 column group l of every token row of the tile.
    pdl_wait();  // the arrival counters are zeroed by the pre-pass kernel in front of this one
    int it = 0;
    while (seg.next(tile, ks0, ks1)) {
      const int buf = it & 1;
      const uint32_t rphase = (it >> 1) & 1;
      ++it;
      if (!mbar_wait_warp(&red_full[buf], rphase, ctl, ST_TIMEOUT_EPILOGUE)) break;
      int b, n0, m0;
      w4_tile_coords(p, tile, MT, b, n0, m0);
      const int rows = min(MT, p.M - m0);
      const float4* h0 = reinterpret_cast<const float4*>(red + (size_t)buf * 2 * Cfg::RED_TILE);
      const float4* h1 = h0 + Cfg::RED_TILE / 4;
      uint16_t* Cout = reinterpret_cast<uint16_t*>(p.C) + (size_t)b * p.M * p.N;
      const int n = n0 + 4 * lane;  // N is a multiple of 8 and n of 4: the four columns are inside N together
      const bool full_tile = (ks0 == 0 && ks1 == p.KS);
      const int my_slot = (ks1 < p.KS) ? 2 * cta + 1 : 2 * cta;
      float4* my_part = reinterpret_cast<float4*>(p.ws_partials + (size_t)my_slot * (MT * W4_BN));
      // Add the two K halves; a whole tile goes straight to C, a split tile's sum to this CTA's partial slot.
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        if (i < rows) {
          const float4 x = h0[i * 32 + lane], y = h1[i * 32 + lane];
          const float4 v = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
          if (!full_tile) my_part[i * 32 + lane] = v;
          else if (n < p.N) w4d_store4<OUT_BF16>(Cout + (size_t)(m0 + i) * p.N + n, v);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&red_empty[buf]);  // the buffer may be refilled
      if (full_tile) continue;

      // Split tile: count arrivals; the last contributor adds all partials in a fixed order.
      const long long first_item = (long long)tile * p.KS;
      const int b_first = w4_owner(T, G, first_item);
      const int b_last = w4_owner(T, G, first_item + p.KS - 1);
      __threadfence();
      __syncwarp();
      uint32_t last = 0;
      if (lane == 0) {
        const uint32_t old = atomicAdd(p.ws_counters + b_first, 1u);
        if (old == (uint32_t)(b_last - b_first)) {
          last = 1;
          p.ws_counters[b_first] = 0;  // every contributor has arrived: leave the counter clean
        }
      }
      last = __shfl_sync(0xffffffffu, last, 0);
      if (!last) continue;
      __threadfence();
      for (int i0 = 0; i0 < rows; i0 += 8) {
        float4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int cc = b_first; cc <= b_last; ++cc) {  // fixed order: results do not depend on arrival order
          const long long c_end = w4_range_begin(T, G, cc + 1);
          const int slot = (c_end >= first_item + p.KS) ? 2 * cc : 2 * cc + 1;
          const float4* part = reinterpret_cast<const float4*>(p.ws_partials + (size_t)slot * (MT * W4_BN));
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (i0 + i < rows) {
              const float4 x = __ldcg(part + (i0 + i) * 32 + lane);
              v[i].x += x.x; v[i].y += x.y; v[i].z += x.z; v[i].w += x.w;
            }
          }
        }
        if (n < p.N) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (i0 + i < rows) w4d_store4<OUT_BF16>(Cout + (size_t)(m0 + i0 + i) * p.N + n, v[i]);
        }
      }
    }
    return;
  }

  // ------------------------------------------------------------------ compute warps
  const int cw = warp - 1;
  const int rb = cw & 7;    // 16-row block of the tile
  const int kh = cw >> 3;   // K half of every slab
  const int g = lane >> 2;  // mma "group id": weight row g / g+8, token g
  const int c = lane & 3;   // mma "thread in group": K pairs and token pairs
  const uint32_t zero = (uint32_t)p.zero;
  const uint32_t sub_lo = (0x6400u + zero) * 0x00010001u;
  const uint32_t sub_hi = ((0x5400u + (zero << 4)) | 0x8000u) * 0x00010001u;
  // Per-thread byte offsets inside a stage, fixed for the whole kernel.  Chunk ch = 4*kh + kc is the
  // 16-byte (32 k) piece of the 128-byte packed row; the activation piece of the same 32 k sits in K block
  // ch/2 at 16-byte position (ch&1)*4 + c of token row g; both tiles are 128-byte swizzled by (row & 7) = g.
  uint32_t w_off[4], a_off[4];
#pragma unroll
  for (int kc = 0; kc < 4; ++kc) {
    const int ch = 4 * kh + kc;
    w_off[kc] = (uint32_t)((16 * rb + g) * 128 + 4 * c + ((ch ^ g) << 4));
    a_off[kc] = (uint32_t)(W4_RAW_BYTES + (ch >> 1) * Cfg::A_KB_BYTES + g * 128 + (((((ch & 1) << 2) + c) ^ g) << 4));
  }
  // scale of this warp's K half: row of the stage's scale tile for chunk kc (groups up to 256 are powers of two)
  const int gshift = 31 - __clz(p.group);
  const bool small_group = p.group <= W4_SLAB_K;
  const uint32_t s_off = (uint32_t)(W4_RAW_PACKED + (16 * rb + g) * 2);
  const float zero4[4] = {0.f, 0.f, 0.f, 0.f};

  int s = 0, it = 0;
  uint32_t phase = 0;
  bool ok = true;
  while (seg.next(tile, ks0, ks1)) {
    float acc[NB][4], acc2[NB][4];  // acc2: second chain when unscaled
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int i = 0; i < 4; ++i) { acc[nb][i] = 0.f; acc2[nb][i] = 0.f; }

    for (int ks = ks0; ks < ks1; ++ks) {
      if (ok) ok = mbar_wait_warp(&full[s], phase, ctl, ST_TIMEOUT_DEQUANT);
      if (ok) {
        const uint8_t* stg = smem + s * Cfg::STAGE_BYTES;
        float pa[NB][4], pb[NB][4];  // two independent accumulation chains per group
#pragma unroll
        for (int kc = 0; kc < 4; ++kc) {
          const uint32_t x_lo = *reinterpret_cast<const uint32_t*>(stg + w_off[kc]);
          const uint32_t x_hi = *reinterpret_cast<const uint32_t*>(stg + w_off[kc] + 8 * 128);
          uint32_t hl[4], hh[4];
          w4d_convert8(x_lo, sub_lo, sub_hi, hl);
          w4d_convert8(x_hi, sub_lo, sub_hi, hh);
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
            const uint4 av = *reinterpret_cast<const uint4*>(stg + a_off[kc] + nb * 8 * 128);
            if constexpr (!SCALED) {
              w4d_mma(acc[nb], hl[0], hh[0], hl[1], hh[1], av.x, av.y, acc[nb]);
              w4d_mma(acc2[nb], hl[2], hh[2], hl[3], hh[3], av.z, av.w, acc2[nb]);
            } else if (kc % FLUSH == 0) {
              w4d_mma(pa[nb], hl[0], hh[0], hl[1], hh[1], av.x, av.y, zero4);
              w4d_mma(pb[nb], hl[2], hh[2], hl[3], hh[3], av.z, av.w, zero4);
            } else {
              w4d_mma(pa[nb], hl[0], hh[0], hl[1], hh[1], av.x, av.y, pa[nb]);
              w4d_mma(pb[nb], hl[2], hh[2], hl[3], hh[3], av.z, av.w, pb[nb]);
            }
          }
          if constexpr (SCALED) {
            if ((kc + 1) % FLUSH == 0) {
              // end of a quantisation group (or of this warp's 128 k of a larger group): scale the partial sums
              const int srow = small_group ? ((kh * 128 + kc * 32) >> gshift) : 0;
              const __half* sp = reinterpret_cast<const __half*>(stg + s_off) + srow * W4_BN;
              const float s_lo = __half2float(sp[0]);
              const float s_hi = __half2float(sp[8]);
#pragma unroll
              for (int nb = 0; nb < NB; ++nb) {
                acc[nb][0] = fmaf(pa[nb][0] + pb[nb][0], s_lo, acc[nb][0]);
                acc[nb][1] = fmaf(pa[nb][1] + pb[nb][1], s_lo, acc[nb][1]);
                acc[nb][2] = fmaf(pa[nb][2] + pb[nb][2], s_hi, acc[nb][2]);
                acc[nb][3] = fmaf(pa[nb][3] + pb[nb][3], s_hi, acc[nb][3]);
              }
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
      }
      if (++s == ST) { s = 0; phase ^= 1u; }
    }
    if constexpr (!SCALED) {
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nb][i] += acc2[nb][i];
    }

    // ---- segment end: hand this warp's K-half sums to the finisher and go on
    const int buf = it & 1;
    const uint32_t ephase = ((it >> 1) & 1) ^ 1u;
    ++it;
    if (ok) ok = mbar_wait_warp(&red_empty[buf], ephase, ctl, ST_TIMEOUT_DEQUANT);
    if (!ok) break;  // an expired wait has set the abort flag: every other wait in the CTA gives up too
    float* r0 = red + (size_t)(buf * 2 + kh) * Cfg::RED_TILE + (2 * c) * W4_BN + 16 * rb + g;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      float* r = r0 + nb * 8 * W4_BN;
      r[0] = acc[nb][0];
      r[W4_BN] = acc[nb][1];
      r[8] = acc[nb][2];
      r[W4_BN + 8] = acc[nb][3];
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&red_full[buf]);
  }
}

}  // namespace qg
