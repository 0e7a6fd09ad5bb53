// Host side of libqgemm.so: argument validation, TMA tensor-map encoding, kernel selection and launch.
// The exported functions are declared and documented in include/qgemm.h.
#include "../../include/qgemm.h"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "w4a16.cuh"
#include "w4a16_decode.cuh"
#include "w4a16_gs.cuh"
#include "act_quant.cuh"
#include "w4a8.cuh"
#include "w8a8.cuh"

namespace {

thread_local char g_err[512] = "";
unsigned long long g_wait_limit_ns = 2000ull * 1000ull * 1000ull;

int fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return -1;
}

#define CUDA_OK(expr)                                                                      \
  do {                                                                                     \
    cudaError_t e_ = (expr);                                                               \
    if (e_ != cudaSuccess) return fail("%s failed: %s", #expr, cudaGetErrorString(e_));   \
  } while (0)

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

constexpr int kMaxDevices = 64;
struct DeviceState {
  bool ready = false;
  int sm_count = 0;
};
std::mutex g_mu;
DeviceState g_dev[kMaxDevices];
EncodeTiledFn g_encode = nullptr;

template <typename K>
int set_smem(K kernel, int bytes) {
  CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  return 0;
}

template <int BN>
int set_smem_w8() {
  using C = qg::W8Cfg<BN>;
  if (set_smem(qg::w8a8_gemm_kernel<BN, false, false>, C::SMEM_BYTES)) return -1;
  if (set_smem(qg::w8a8_gemm_kernel<BN, false, true>, C::SMEM_BYTES)) return -1;
  if (set_smem(qg::w8a8_gemm_kernel<BN, true, false>, C::SMEM_BYTES)) return -1;
  if (set_smem(qg::w8a8_gemm_kernel<BN, true, true>, C::SMEM_BYTES)) return -1;
  if (set_smem(qg::w8a8_gemm_kernel<BN, true, false, true>, C::SMEM_BYTES)) return -1;
  if (set_smem(qg::w8a8_gemm_kernel<BN, true, true, true>, C::SMEM_BYTES)) return -1;
  if (BN == 256) {  // the two-CTA K split
    if (set_smem(qg::w8a8_gemm_kernel<256, false, false, false, true>, C::SMEM_BYTES)) return -1;
    if (set_smem(qg::w8a8_gemm_kernel<256, false, true, false, true>, C::SMEM_BYTES)) return -1;
    if (set_smem(qg::w8a8_gemm_kernel<256, true, false, false, true>, C::SMEM_BYTES)) return -1;
    if (set_smem(qg::w8a8_gemm_kernel<256, true, true, false, true>, C::SMEM_BYTES)) return -1;
  }
  return 0;
}
template <int FLUSH>
int set_smem_w4d() {
  if (set_smem(qg::w4a16_decode_kernel<FLUSH, 1, false>, qg::W4DCfg<1>::SMEM_BYTES)) return -1;
  if (set_smem(qg::w4a16_decode_kernel<FLUSH, 1, true>, qg::W4DCfg<1>::SMEM_BYTES)) return -1;
  if (set_smem(qg::w4a16_decode_kernel<FLUSH, 2, false>, qg::W4DCfg<2>::SMEM_BYTES)) return -1;
  if (set_smem(qg::w4a16_decode_kernel<FLUSH, 2, true>, qg::W4DCfg<2>::SMEM_BYTES)) return -1;
  return 0;
}
template <int MT>
int set_smem_w4i8() {
  using C = qg::W4I8Cfg<MT>;
  if (set_smem(qg::w4a8_gemm_kernel<MT, false>, C::SMEM_BYTES)) return -1;
  if (set_smem(qg::w4a8_gemm_kernel<MT, true>, C::SMEM_BYTES)) return -1;
  return 0;
}
template <int MT>
int set_smem_w4() {
  using C = qg::W4Cfg<MT>;
  if (set_smem(qg::w4a16_gemm_kernel<MT, false>, C::SMEM_BYTES)) return -1;
  if (set_smem(qg::w4a16_gemm_kernel<MT, true>, C::SMEM_BYTES)) return -1;
  return 0;
}

template <int MT>
int set_smem_w4g() {
  using C = qg::W4GCfg<MT>;
  if (set_smem(qg::w4a16_gs_kernel<MT, false>, C::SMEM_BYTES)) return -1;
  if (set_smem(qg::w4a16_gs_kernel<MT, true>, C::SMEM_BYTES)) return -1;
  if (set_smem(qg::w4a16_gs_kernel<MT, false, true>, C::SMEM_BYTES)) return -1;
  if (set_smem(qg::w4a16_gs_kernel<MT, true, true>, C::SMEM_BYTES)) return -1;
  if (set_smem(qg::w4a16_gs_kernel<MT, false, false, true>, C::SMEM_BYTES)) return -1;
  if (set_smem(qg::w4a16_gs_kernel<MT, true, false, true>, C::SMEM_BYTES)) return -1;
  if constexpr (MT == 16) {
    if (set_smem(qg::w4a16_gs_kernel<16, false, false, false, true>, C::SMEM_BYTES)) return -1;
    if (set_smem(qg::w4a16_gs_kernel<16, true, false, false, true>, C::SMEM_BYTES)) return -1;
  }
  return 0;
}

// Once per device, with that device current.
int ensure_device(int* sm_count) {
  int dev = 0;
  CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail("device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_mu);
  DeviceState& st = g_dev[dev];
  if (!st.ready) {
    cudaDeviceProp prop;
    CUDA_OK(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10) return fail("libqgemm needs an sm_100a device (B200); device %d is sm_%d%d", dev, prop.major, prop.minor);
    if (g_encode == nullptr) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qres;
      CUDA_OK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
      if (qres != cudaDriverEntryPointSuccess || fn == nullptr) return fail("cuTensorMapEncodeTiled not available from the driver");
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    if (set_smem_w8<128>() || set_smem_w8<256>()) return -1;
    if (set_smem_w4<16>() || set_smem_w4<32>() || set_smem_w4<64>() || set_smem_w4<128>()) return -1;
    if (set_smem_w4g<16>() || set_smem_w4g<32>() || set_smem_w4g<64>()) return -1;
    if (set_smem_w4i8<16>() || set_smem_w4i8<32>() || set_smem_w4i8<64>() || set_smem_w4i8<128>()) return -1;
    if (set_smem_w4d<0>() || set_smem_w4d<1>() || set_smem_w4d<2>() || set_smem_w4d<4>()) return -1;
    st.sm_count = prop.multiProcessorCount;
    st.ready = true;
  }
  *sm_count = st.sm_count;
  return 0;
}

// rank-2/3 row-major tensor map; dims/box innermost first; strides in bytes for dims 1.. (innermost is dense).
int encode_map(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
               const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz) {
  cuuint64_t gdim[3], gstr[2];
  cuuint32_t bx[3], es[3];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i > 0) gstr[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = g_encode(map, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bx, es,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Launch `kernel` so that it may start while the kernel in front of it on the stream is still running
// (programmatic dependent launch); the kernel itself waits before it reads that kernel's results.
// QGEMM_PDL=0 falls back to plain stream order.
template <typename... KArgs, typename... Args>
int launch_pdl(void (*kernel)(KArgs...), int grid, int threads, int smem, cudaStream_t s, Args&&... args) {
  static const int pdl = getenv("QGEMM_PDL") ? atoi(getenv("QGEMM_PDL")) : 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...));
  return 0;
}

// Rasterisation band: the tiles of `group_m` consecutive row blocks are walked column block by column block, so a
// wave of CTAs shares few B tiles and the band's A rows (group_m x 128 x K bytes) stay in L2 while every B tile
// streams through once per band.  As many row blocks as keep the band's A rows within 34 MB, at least 8: config 3
// takes all 32 row blocks (16.8 MB, B read from DRAM once instead of four times: 172 -> 165 us; 16 or 24 row blocks:
// 170 us), the f16 GEMM of 4096 x 8192 x 28672 takes 16 (33.5 MB: 1525 us; 8: 1570, 32: 1553).
int w8_group_m(int64_t m_tiles, int64_t k_bytes) {
  static const int forced = getenv("QGEMM_W8_GROUP_M") ? atoi(getenv("QGEMM_W8_GROUP_M")) : 0;  // tuning override
  int64_t g = forced > 0 ? forced : (34ll << 20) / (128 * (k_bytes > 0 ? k_bytes : 1));
  if (g < 8) g = 8;
  if (g > m_tiles) g = m_tiles;
  return (int)(g > 0 ? g : 1);
}

template <int BN, bool NK, bool BF>
int launch_w8(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const qg::W8A8Params& p, int grid,
              cudaStream_t s) {
  qg::W8Dst dst;
  for (int d = 0; d < 8; ++d) dst.m[d] = tmC;
  qg::w8a8_gemm_kernel<BN, NK, BF><<<grid, qg::W8_THREADS, qg::W8Cfg<BN>::SMEM_BYTES, s>>>(tmA, tmB, dst, p);
  CUDA_OK(cudaGetLastError());
  return 0;
}

// The K split: clusters of two CTAs, one 128 x 256 tile per cluster.
template <bool NK, bool BF>
int launch_w8_splitk(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const qg::W8A8Params& p,
                     int tiles, cudaStream_t s) {
  qg::W8Dst dst;
  for (int d = 0; d < 8; ++d) dst.m[d] = tmC;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * tiles));
  cfg.blockDim = dim3((unsigned)qg::W8_THREADS);
  cfg.dynamicSmemBytes = (size_t)qg::W8Cfg<256>::SMEM_BYTES;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CUDA_OK(cudaLaunchKernelEx(&cfg, qg::w8a8_gemm_kernel<256, NK, BF, false, true>, tmA, tmB, dst, p));
  return 0;
}

template <int MT>
int launch_w4(bool bf, const CUtensorMap& tmW, const CUtensorMap& tmS, const CUtensorMap& tmA,
              const qg::W4A16Params& p, int grid, cudaStream_t s) {
  if (bf) return launch_pdl(qg::w4a16_gemm_kernel<MT, true>, grid, qg::W4_THREADS, qg::W4Cfg<MT>::SMEM_BYTES, s, tmW, tmS, tmA, p);
  return launch_pdl(qg::w4a16_gemm_kernel<MT, false>, grid, qg::W4_THREADS, qg::W4Cfg<MT>::SMEM_BYTES, s, tmW, tmS, tmA, p);
}
// Test hook (qgemm_debug_withhold_commit): see W4GDebug.
int g_w4g_withhold_commit = 0;

// `tmZ` non-null: the zeros-tensor instantiation (not combined with the gathered form).
template <int MT>
int launch_w4g(bool bf, const CUtensorMap& tmW, const CUtensorMap& tmS, const CUtensorMap* tmZ, const CUtensorMap& tmA,
               const qg::W4A16Params& p, int grid, cudaStream_t s) {
  qg::W4GDebug dbg;
  dbg.withhold_last_commit = g_w4g_withhold_commit;
  constexpr int smem = qg::W4GCfg<MT>::SMEM_BYTES;
  if (tmZ != nullptr) {
    if (bf) return launch_pdl(qg::w4a16_gs_kernel<MT, true, false, true>, grid, qg::W4G_THREADS, smem, s, tmW, tmS, *tmZ, tmA, p, dbg);
    return launch_pdl(qg::w4a16_gs_kernel<MT, false, false, true>, grid, qg::W4G_THREADS, smem, s, tmW, tmS, *tmZ, tmA, p, dbg);
  }
  if (p.n_dst > 0) {
    if (bf) return launch_pdl(qg::w4a16_gs_kernel<MT, true, true>, grid, qg::W4G_THREADS, smem, s, tmW, tmS, tmS, tmA, p, dbg);
    return launch_pdl(qg::w4a16_gs_kernel<MT, false, true>, grid, qg::W4G_THREADS, smem, s, tmW, tmS, tmS, tmA, p, dbg);
  }
  if (bf) return launch_pdl(qg::w4a16_gs_kernel<MT, true>, grid, qg::W4G_THREADS, smem, s, tmW, tmS, tmS, tmA, p, dbg);
  return launch_pdl(qg::w4a16_gs_kernel<MT, false>, grid, qg::W4G_THREADS, smem, s, tmW, tmS, tmS, tmA, p, dbg);
}

// Single-launch form of the group-sum kernel (see its SMALL parameter): clusters of `cluster` CTAs, one tile per cluster,
// no pre-pass in front.  Still a programmatic dependent of whatever is in front of it on the stream.
int launch_w4g_small(bool bf, const CUtensorMap& tmW, const CUtensorMap& tmS, const CUtensorMap& tmA,
                     const qg::W4A16Params& p, int grid, int cluster, cudaStream_t s) {
  static const int pdl = getenv("QGEMM_PDL") ? atoi(getenv("QGEMM_PDL")) : 1;
  qg::W4GDebug dbg;
  dbg.withhold_last_commit = g_w4g_withhold_commit;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)qg::W4G_THREADS);
  cfg.dynamicSmemBytes = (size_t)qg::W4GCfg<16>::SMEM_BYTES;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 2 : 1;
  if (bf) CUDA_OK(cudaLaunchKernelEx(&cfg, qg::w4a16_gs_kernel<16, true, false, false, true>, tmW, tmS, tmS, tmA, p, dbg));
  else CUDA_OK(cudaLaunchKernelEx(&cfg, qg::w4a16_gs_kernel<16, false, false, false, true>, tmW, tmS, tmS, tmA, p, dbg));
  return 0;
}

// The group-sum kernel (w4a16_gs.cuh) serves up to 64 tokens when the scale groups are 128 wide, a multiple of
// 256 or the whole K (or there are no scales); it is faster than the register-operand decode kernel at every
// token count (K=8192, N=28672: 36 against 40 us at one token, 37 against 42 us at eight).  Groups of 32 / 64 keep
// the decode kernel (M <= 8) and the per-weight-scale tcgen05 kernel.  QGEMM_W4_GS=0 disables the group-sum kernel,
// QGEMM_W4_GS_MIN_M raises the token count from which it is used.
int w4_gs_min_m() {
  static const int v = getenv("QGEMM_W4_GS_MIN_M") ? atoi(getenv("QGEMM_W4_GS_MIN_M")) : 1;
  return v;
}
bool w4_gs_shape_ok(int64_t M, bool has_scales, int64_t group, int64_t K) {
  static const int enabled = getenv("QGEMM_W4_GS") ? atoi(getenv("QGEMM_W4_GS")) : 1;
  if (!enabled || M > 64 || M < w4_gs_min_m()) return false;
  return !has_scales || group == 128 || group % 256 == 0 || group >= K;
}

template <int FLUSH, int NB>
int launch_w4d_nb(bool bf, const CUtensorMap& tmW, const CUtensorMap& tmS, const CUtensorMap& tmA,
                  const qg::W4A16Params& p, int grid, cudaStream_t s) {
  if (bf) return launch_pdl(qg::w4a16_decode_kernel<FLUSH, NB, true>, grid, qg::W4D_THREADS, qg::W4DCfg<NB>::SMEM_BYTES, s, tmW, tmS, tmA, p);
  return launch_pdl(qg::w4a16_decode_kernel<FLUSH, NB, false>, grid, qg::W4D_THREADS, qg::W4DCfg<NB>::SMEM_BYTES, s, tmW, tmS, tmA, p);
}
template <int FLUSH>
int launch_w4d(bool bf, int mt, const CUtensorMap& tmW, const CUtensorMap& tmS, const CUtensorMap& tmA,
               const qg::W4A16Params& p, int grid, cudaStream_t s) {
  if (mt == 16) return launch_w4d_nb<FLUSH, 2>(bf, tmW, tmS, tmA, p, grid, s);
  return launch_w4d_nb<FLUSH, 1>(bf, tmW, tmS, tmA, p, grid, s);
}
// Token counts up to this use the register-operand streaming kernel (w4a16_decode.cuh); above it the
// tcgen05 kernel (w4a16.cuh).
int w4_decode_max_m() {
  static int v = -1;
  if (v < 0) {
    v = 8;
    if (const char* e = getenv("QGEMM_W4_DECODE_MAX_M")) v = atoi(e) < 16 ? atoi(e) : 16;
  }
  return v;
}
bool w4_use_decode(int64_t M) { return M <= w4_decode_max_m(); }
// Token-tile height: 8 for the decode kernel, 16..128 for the tcgen05 kernel.
// Token-tile height: 16 / 32 for the group-sum kernel, 8 for the decode kernel, 16..128 for the tcgen05 kernel.
int w4_pick_mt(int64_t M, bool gs) {
  if (gs) return M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  if (w4_use_decode(M)) return M <= 8 ? 8 : 16;
  return M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
}

constexpr int64_t kW4MaxGrid = 1024;
constexpr int64_t kW4CounterBytes = kW4MaxGrid * 4;

__global__ void unpack_int4_kernel(const uint8_t* __restrict__ packed, int8_t* __restrict__ out, long long n_bytes,
                                   int signed_nibbles) {
  // 16 packed bytes -> 32 int8 values per thread; low nibble first.
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long base = i * 16;
  if (base >= n_bytes) return;
  if (base + 16 <= n_bytes) {
    const uint4 v = *reinterpret_cast<const uint4*>(packed + base);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t lo = w[j] & 0x0f0f0f0fu;         // even elements
      uint32_t hi = (w[j] >> 4) & 0x0f0f0f0fu;  // odd elements
      if (signed_nibbles) {                     // two's complement nibble: (x ^ 8) - 8 per byte
        lo = __vsub4(lo ^ 0x08080808u, 0x08080808u);
        hi = __vsub4(hi ^ 0x08080808u, 0x08080808u);
      }
      o[2 * j] = __byte_perm(lo, hi, 0x5140);      // e0 o0 e1 o1
      o[2 * j + 1] = __byte_perm(lo, hi, 0x7362);  // e2 o2 e3 o3
    }
    uint4* dst = reinterpret_cast<uint4*>(out + base * 2);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  } else {
    for (long long b = base; b < n_bytes; ++b) {
      int lo = packed[b] & 0xF, hi = packed[b] >> 4;
      if (signed_nibbles) {
        lo = (lo ^ 8) - 8;
        hi = (hi ^ 8) - 8;
      }
      out[2 * b] = (int8_t)lo;
      out[2 * b + 1] = (int8_t)hi;
    }
  }
}

}  // namespace

template <int MT>
static int launch_w4i8(bool sgn, const CUtensorMap& tmW, const CUtensorMap& tmA, const qg::W4A8Params& p, int grid,
                       cudaStream_t s) {
  if (sgn) return launch_pdl(qg::w4a8_gemm_kernel<MT, true>, grid, qg::W4_THREADS, qg::W4I8Cfg<MT>::SMEM_BYTES, s, tmW, tmA, p);
  return launch_pdl(qg::w4a8_gemm_kernel<MT, false>, grid, qg::W4_THREADS, qg::W4I8Cfg<MT>::SMEM_BYTES, s, tmW, tmA, p);
}

// Fused path of qgemm_w4a8 for up to 128 tokens: no int8 copy of the weights; the caller's [N, K] workspace
// only holds the small scratch (arrival counters, int32 partial sums, reordered activations, row sums).
// Returns 1 when the problem does not qualify (the caller then takes the two-kernel path).
// `A` int8 [M, K]; or, with `X` non-null, bf16 / f16 activations that the pre-pass quantises per token itself
// (scales to `scale_out`).
static int w4a8_fused(const int8_t* A, const uint8_t* qB, int8_t* workspace, int* C, int64_t M, int64_t N, int64_t K,
                      int signed_nibbles, uint32_t* status, cudaStream_t s, const void* X = nullptr, int x_is_bf16 = 0,
                      int round_scale = 0, float* scale_out = nullptr) {
  static const int enabled = getenv("QGEMM_W4A8_FUSED") ? atoi(getenv("QGEMM_W4A8_FUSED")) : 1;
  if (!enabled || M > 128 || !aligned16(workspace)) return 1;
  int sms = 0;
  if (ensure_device(&sms)) return -1;
  const int mt = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  const int64_t grid_max = sms < kW4MaxGrid ? sms : kW4MaxGrid;
  const int64_t partial_bytes = grid_max * 2 * (int64_t)mt * 128 * 4;
  const int64_t a_bytes = ((M * K + 255) / 256) * 256;
  const int64_t need = kW4CounterBytes + partial_bytes + a_bytes + ((M * 4 + 255) / 256) * 256;
  if (need > N * K) return 1;  // the caller's workspace is [N, K] int8
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  uint8_t* a_prepared = ws + kW4CounterBytes + partial_bytes;
  int* row_sums = reinterpret_cast<int*>(a_prepared + a_bytes);

  CUtensorMap tmW, tmA;
  {
    const uint64_t dims[2] = {(uint64_t)(K / 2), (uint64_t)N};
    const uint64_t str[1] = {(uint64_t)(K / 2)};
    const uint32_t box[2] = {128, 128};
    if (encode_map(&tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, qB, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
  }
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    const uint64_t str[1] = {(uint64_t)K};
    const uint32_t box[2] = {128, (uint32_t)mt};
    if (encode_map(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a_prepared, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
  }
  qg::W4A8Params p;
  p.C = C;
  p.ws_counters = reinterpret_cast<uint32_t*>(ws);
  p.ws_partials = reinterpret_cast<int*>(ws + kW4CounterBytes);
  p.row_sums = row_sums;
  p.M = (int)M;
  p.N = (int)N;
  p.K = (int)K;
  p.n_tiles = (int)((N + 127) / 128);
  p.KS = (int)((K + 255) / 256);
  p.total_items = (long long)p.n_tiles * p.KS;
  p.status = status;
  p.wait_limit_ns = g_wait_limit_ns;
  int64_t grid = grid_max < p.total_items ? grid_max : p.total_items;
  // a programmatic dependent of whatever is in front: behind another call of this operator it is resident early
  if (X != nullptr) {
    if (launch_pdl(qg::w4a8_quant_prepare_activations, (int)M, 256, 0, s, static_cast<const uint4*>(X), x_is_bf16,
                   round_scale, reinterpret_cast<uint2*>(a_prepared), row_sums, scale_out,
                   reinterpret_cast<uint32_t*>(ws), (int)(kW4CounterBytes / 4), (int)K))
      return -1;
  } else if (launch_pdl(qg::w4a8_prepare_activations, (int)M, 256, 0, s, reinterpret_cast<const uint2*>(A),
                        reinterpret_cast<uint2*>(a_prepared), row_sums, reinterpret_cast<uint32_t*>(ws),
                        (int)(kW4CounterBytes / 4), (int)K))
    return -1;
  const bool sgn = signed_nibbles != 0;
  switch (mt) {
    case 16: return launch_w4i8<16>(sgn, tmW, tmA, p, (int)grid, s);
    case 32: return launch_w4i8<32>(sgn, tmW, tmA, p, (int)grid, s);
    case 64: return launch_w4i8<64>(sgn, tmW, tmA, p, (int)grid, s);
    default: return launch_w4i8<128>(sgn, tmW, tmA, p, (int)grid, s);
  }
}

extern "C" {

int qgemm_version(void) { return 1006; }  // 1.6: + in-flight zero tensors, W4A8 with the activation quantiser fused into its pre-pass

const char* qgemm_last_error(void) { return g_err; }

void qgemm_set_wait_limit_ms(uint32_t ms) { g_wait_limit_ns = (unsigned long long)ms * 1000000ull; }

void qgemm_debug_withhold_commit(int on) { g_w4g_withhold_commit = (on == 2) ? 2 : (on ? 1 : 0); }

int qgemm_init(void) {
  int sms = 0;
  return ensure_device(&sms);
}

// Plain / batched form: meta == nullptr.  Grouped form: A and C are single [M, K] / [M, N] stacks, B holds
// `batch` (= groups) matrices and `meta` lists num_blocks row blocks (group, first row, valid rows).
static int w8a8_impl(const int8_t* A, const int8_t* B, const float* scale_b, const float* scale_a, void* C,
                     int32_t* acc_out, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t scale_b_len,
                     int64_t scale_a_len, int out_dtype, int b_layout, uint32_t* status, void* stream,
                     const int* meta, int64_t num_blocks) {
  const int64_t batchA = meta ? 1 : batch;  // batch extent of A, C and scale_a
  if (batch <= 0 || M <= 0 || N <= 0 || K <= 0) return fail("qgemm_w8a8: batch, M, N, K must be positive (got %lld, %lld, %lld, %lld)", (long long)batch, (long long)M, (long long)N, (long long)K);
  if (M > (1ll << 30) || N > (1ll << 30) || K > (1ll << 30) || batch > 65535) return fail("qgemm_w8a8: dimension too large");
  if (A == nullptr || B == nullptr) return fail("qgemm_w8a8: A and B must not be null");
  if (b_layout != QGEMM_B_KN && b_layout != QGEMM_B_NK) return fail("qgemm_w8a8: unknown b_layout %d", b_layout);
  if (out_dtype == QGEMM_DT_I32) {
    if (C == nullptr) return fail("qgemm_w8a8: int32 output needs C");
    if (acc_out != nullptr) return fail("qgemm_w8a8: with int32 output pass the buffer as C and acc_out = NULL");
    acc_out = static_cast<int32_t*>(C);
    C = nullptr;
  } else if (out_dtype == QGEMM_DT_F16 || out_dtype == QGEMM_DT_BF16) {
    if (C == nullptr && acc_out == nullptr) return fail("qgemm_w8a8: neither C nor acc_out given");
    if (C != nullptr) {
      if (scale_b == nullptr) return fail("qgemm_w8a8: scale_b must not be null");
      if (scale_b_len != 1 && scale_b_len != N && scale_b_len != batch * N) return fail("qgemm_w8a8: scale_b_len must be 1, N or batch*N (got %lld)", (long long)scale_b_len);
      if (scale_a != nullptr && scale_a_len != M && scale_a_len != batchA * M) return fail("qgemm_w8a8: scale_a_len must be M or batch*M (got %lld)", (long long)scale_a_len);
    }
  } else {
    return fail("qgemm_w8a8: out_dtype must be F16, BF16 or I32 (got %d)", out_dtype);
  }
  if (K % 16 != 0 || N % 16 != 0) return fail("qgemm_w8a8: K and N must be multiples of 16 (got K=%lld, N=%lld)", (long long)K, (long long)N);
  if (!aligned16(A) || !aligned16(B) || !aligned16(C) || !aligned16(acc_out)) return fail("qgemm_w8a8: A, B, C and acc_out must be 16-byte aligned");

  int sms = 0;
  if (ensure_device(&sms)) return -1;

  CUtensorMap tmA, tmB;
  {
    const uint64_t dims[3] = {(uint64_t)K, (uint64_t)M, (uint64_t)batchA};
    const uint64_t str[2] = {(uint64_t)K, (uint64_t)M * (uint64_t)K};
    const uint32_t box[3] = {128, 128, 1};
    if (encode_map(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, A, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
  }
  const int64_t m_tiles = meta ? num_blocks : (M + 127) / 128;
  const int64_t tiles256 = batchA * m_tiles * ((N + 255) / 256);
  // Fewer 256-wide tiles than half the SMs: split K over pairs of CTAs (one tile per pair, twice as many SMs at
  // work on full-width tiles) instead of falling back to 128-wide tiles - when K is long enough to pay for the
  // cluster launch and the exchange: on 2 x 512 x K x 2048, split against 128-wide tiles, K = 7168: 19.8 / 23.6 us,
  // 4096: 14.9 / 16.2, 3072: 13.7 / 13.3, and 256 x 1024 x 1024: 9.9 / 7.0, so the split starts at K = 4096.
  // QGEMM_W8_SPLITK=0 disables it.
  static const int splitk_on = getenv("QGEMM_W8_SPLITK") ? atoi(getenv("QGEMM_W8_SPLITK")) : 1;
  const bool use_splitk = splitk_on && meta == nullptr && N > 128 && 2 * tiles256 <= sms && (K + 127) / 128 >= 32;
  const int BN = (N > 128 && (tiles256 >= sms || use_splitk)) ? 256 : 128;
  // Width actually computed per tile (a multiple of 32, at most BN).  Narrower tiles that fill the last
  // round of the persistent grid better were measured slower on B200 (224 instead of 256 columns on the
  // 4096 x 4096 x 14336 shape: 235 us against 231 us), so the full width is used.
  const int bn_eff = BN;
  if (b_layout == QGEMM_B_KN) {
    const uint64_t dims[3] = {(uint64_t)N, (uint64_t)K, (uint64_t)batch};
    const uint64_t str[2] = {(uint64_t)N, (uint64_t)K * (uint64_t)N};
    const uint32_t box[3] = {128, 128, 1};
    if (encode_map(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, B, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
  } else {
    const uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, (uint64_t)batch};
    const uint64_t str[2] = {(uint64_t)K, (uint64_t)N * (uint64_t)K};
    const uint32_t box[3] = {128, (uint32_t)BN, 1};
    if (encode_map(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, B, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
  }

  // C as a tensor map for the epilogue's tiled stores: boxes of 64 outputs x 32 rows, 128-byte swizzle.
  CUtensorMap tmC = tmA;
  static const int tma_store_on = getenv("QGEMM_W8_TMA_STORE") ? atoi(getenv("QGEMM_W8_TMA_STORE")) : 1;  // 0: per-row stores
  const bool tma_store = tma_store_on && C != nullptr && (bn_eff % 64) == 0;
  if (tma_store) {
    const uint64_t dims[3] = {(uint64_t)N, (uint64_t)M, (uint64_t)batchA};
    const uint64_t str[2] = {(uint64_t)N * 2, (uint64_t)M * (uint64_t)N * 2};
    const uint32_t box[3] = {64, 32, 1};
    if (encode_map(&tmC, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, C, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
  }

  qg::W8A8Params p;
  p.tma_store = tma_store ? 1 : 0;
  p.n_dst = 0;
  p.col0 = 0;
  p.scale_b = scale_b;
  p.scale_a = scale_a;
  p.C = C;
  p.acc_out = acc_out;
  p.batch = (int)batchA;
  p.meta = meta;
  p.groups = (int)batch;
  p.M = (int)M;
  p.N = (int)N;
  p.K = (int)K;
  p.sb_mode = (scale_b_len == 1) ? 0 : ((scale_b_len == N) ? 1 : 2);
  p.sa_mode = (scale_a == nullptr) ? 0 : ((scale_a_len == M) ? 1 : 2);
  p.m_tiles = (int)m_tiles;
  p.group_m = w8_group_m(m_tiles, K);
  p.n_tiles = (int)((N + bn_eff - 1) / bn_eff);
  p.bn = bn_eff;
  const int64_t num_tiles = batchA * p.m_tiles * p.n_tiles;
  if (num_tiles > 0x7fffffff) return fail("qgemm_w8a8: too many tiles");
  p.num_tiles = (int)num_tiles;
  p.k_blocks = (int)((K + 127) / 128);
  p.status = status;
  p.wait_limit_ns = g_wait_limit_ns;
  const int grid = (int)(num_tiles < sms ? num_tiles : sms);
  // Tail split: when the last round of the persistent grid would run R < grid/2 tiles, those tiles are issued
  // as 2R half-width items instead ([K, N] layout, 256-column tiles).
  p.split_from = p.num_items = p.num_tiles;
  {
    static const int tail_split = getenv("QGEMM_W8_TAIL_SPLIT") ? atoi(getenv("QGEMM_W8_TAIL_SPLIT")) : 1;
    const int64_t R = num_tiles % grid;
    if (tail_split && b_layout == QGEMM_B_KN && BN == 256 && num_tiles > grid && R > 0 && 2 * R <= grid) {
      p.split_from = (int)(num_tiles - R);
      p.num_items = (int)(num_tiles + R);
    }
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool nk = b_layout == QGEMM_B_NK;
  const bool bf = out_dtype == QGEMM_DT_BF16;
  if (use_splitk) {
    if (nk) return bf ? launch_w8_splitk<true, true>(tmA, tmB, tmC, p, (int)num_tiles, s) : launch_w8_splitk<true, false>(tmA, tmB, tmC, p, (int)num_tiles, s);
    return bf ? launch_w8_splitk<false, true>(tmA, tmB, tmC, p, (int)num_tiles, s) : launch_w8_splitk<false, false>(tmA, tmB, tmC, p, (int)num_tiles, s);
  }
  if (BN == 256) {
    if (nk) return bf ? launch_w8<256, true, true>(tmA, tmB, tmC, p, grid, s) : launch_w8<256, true, false>(tmA, tmB, tmC, p, grid, s);
    return bf ? launch_w8<256, false, true>(tmA, tmB, tmC, p, grid, s) : launch_w8<256, false, false>(tmA, tmB, tmC, p, grid, s);
  }
  if (nk) return bf ? launch_w8<128, true, true>(tmA, tmB, tmC, p, grid, s) : launch_w8<128, true, false>(tmA, tmB, tmC, p, grid, s);
  return bf ? launch_w8<128, false, true>(tmA, tmB, tmC, p, grid, s) : launch_w8<128, false, false>(tmA, tmB, tmC, p, grid, s);
}

int qgemm_w8a8(const int8_t* A, const int8_t* B, const float* scale_b, const float* scale_a, void* C,
               int32_t* acc_out, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t scale_b_len,
               int64_t scale_a_len, int out_dtype, int b_layout, uint32_t* status, void* stream) {
  return w8a8_impl(A, B, scale_b, scale_a, C, acc_out, batch, M, N, K, scale_b_len, scale_a_len, out_dtype, b_layout,
                   status, stream, nullptr, 0);
}

int qgemm_w8a8_grouped(const int8_t* A, const int8_t* B, const float* scale_b, const float* scale_a, void* C,
                       int32_t* acc_out, const int32_t* block_metadata, int64_t num_blocks, int64_t groups,
                       int64_t total_M, int64_t N, int64_t K, int64_t scale_b_len, int64_t scale_a_len, int out_dtype,
                       int b_layout, uint32_t* status, void* stream) {
  if (num_blocks < 0) return fail("qgemm_w8a8_grouped: num_blocks must not be negative (got %lld)", (long long)num_blocks);
  if (num_blocks == 0 || total_M == 0) return 0;  // no rows: nothing to compute
  if (block_metadata == nullptr) return fail("qgemm_w8a8_grouped: block_metadata must not be null");
  if ((reinterpret_cast<uintptr_t>(block_metadata) & 3u) != 0) return fail("qgemm_w8a8_grouped: block_metadata must be 4-byte aligned");
  if (num_blocks > (1ll << 24)) return fail("qgemm_w8a8_grouped: too many row blocks (%lld)", (long long)num_blocks);
  return w8a8_impl(A, B, scale_b, scale_a, C, acc_out, groups, total_M, N, K, scale_b_len, scale_a_len, out_dtype,
                   b_layout, status, stream, block_metadata, num_blocks);
}

int64_t qgemm_w4a16_counter_bytes(void) { return kW4CounterBytes; }

// Token counts from this on (and N a multiple of 16) dequantise the whole weight matrix to f16 once and run
// the f16 tensor-core GEMM on it: the in-flight conversion is repeated for every 128-token tile and at some point
// costs more than writing and re-reading 2 bytes per weight.  Measured sweep on K=8192, N=28672 (in-flight against
// dequantise-once, us): 512 tokens 230 / 366, 1024: 445 / 526, 1536: 685 / 710, 2048: 927 / 877 - the paths cross
// near 1800.  QGEMM_W4_GEMM_MIN_M overrides the threshold (0 = never).
int64_t w4_gemm_min_m() {
  static int64_t v = -1;
  if (v < 0) {
    v = 1792;
    if (const char* e = getenv("QGEMM_W4_GEMM_MIN_M")) v = atoll(e) > 0 ? atoll(e) : (1ll << 62);
    if (v <= 16) v = 17;  // the small-token kernels keep their range
  }
  return v;
}
bool w4_use_f16_gemm(int64_t M, int64_t N) { return M >= w4_gemm_min_m() && (N % 16) == 0; }

static int64_t w4_workspace_bytes(int64_t batch, int64_t M, int64_t N, int64_t K, bool dequant_once) {
  int sms = 0;
  if (ensure_device(&sms)) return -1;
  const int64_t grid = sms < kW4MaxGrid ? sms : kW4MaxGrid;
  // sized for whichever small-token kernel the scale groups will select (the group-sum kernel's tile is the taller)
  const int mt = M <= 64 ? w4_pick_mt(M, true) : w4_pick_mt(M, false);
  // the arrival counters first (fixed place whatever the tile height), then two partial slots of
  // [MT][128] fp32 per CTA, then the f16 copy of the activations in the kernel's K order
  // ... and, for the large-token path, the dequantised f16 weights
  return kW4CounterBytes + grid * 2 * (int64_t)mt * 128 * 4 + batch * M * K * 2 +
         ((dequant_once || w4_use_f16_gemm(M, N)) ? batch * N * K * 2 : 0);
}

int64_t qgemm_w4a16_batched_workspace_bytes(int64_t batch, int64_t M, int64_t N, int64_t K) {
  return w4_workspace_bytes(batch, M, N, K, false);
}

int64_t qgemm_w4a16_ex_workspace_bytes(int64_t batch, int64_t M, int64_t N, int64_t K, int has_zeros_tensor) {
  return w4_workspace_bytes(batch, M, N, K, has_zeros_tensor != 0);
}

int64_t qgemm_w4a16_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  return qgemm_w4a16_batched_workspace_bytes(1, M, N, K);
}

// Destinations of the gathered form: `n` row-major [M, ldc] buffers (one per rank, peers' buffers mapped into this
// process), this rank's columns starting at col0.
struct GatherDst {
  void* const* dst;
  int n;
  int64_t ldc, col0;
};

// C[b] = A16[b] (f16 [M, K]) x W16[b]^T (f16 [N, K]), fp32 accumulation, f16 / bf16 out: the tile pipeline of
// the W8A8 kernel on 2-byte elements (K counted in bytes).
static int w4_f16_gemm(const void* A16, const void* W16, void* C, int64_t batch, int64_t M, int64_t N, int64_t K,
                       bool bf, uint32_t* status, cudaStream_t s, int sms, const GatherDst* gd) {
  const int64_t Kb = K * 2;
  CUtensorMap tmA, tmB, tmC;
  {
    const uint64_t dims[3] = {(uint64_t)Kb, (uint64_t)M, (uint64_t)batch};
    const uint64_t str[2] = {(uint64_t)Kb, (uint64_t)M * (uint64_t)Kb};
    const uint32_t box[3] = {128, 128, 1};
    if (encode_map(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, A16, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
  }
  const int64_t m_tiles = (M + 127) / 128;
  const int BN = (N > 128 && batch * m_tiles * ((N + 255) / 256) >= sms) ? 256 : 128;
  {
    const uint64_t dims[3] = {(uint64_t)Kb, (uint64_t)N, (uint64_t)batch};
    const uint64_t str[2] = {(uint64_t)Kb, (uint64_t)N * (uint64_t)Kb};
    const uint32_t box[3] = {128, (uint32_t)BN, 1};
    if (encode_map(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, W16, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
  }
  qg::W8Dst dst;
  if (gd == nullptr) {
    const uint64_t dims[3] = {(uint64_t)N, (uint64_t)M, (uint64_t)batch};
    const uint64_t str[2] = {(uint64_t)N * 2, (uint64_t)M * (uint64_t)N * 2};
    const uint32_t box[3] = {64, 32, 1};
    if (encode_map(&tmC, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, C, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    for (int d = 0; d < 8; ++d) dst.m[d] = tmC;
  } else {
    // one map per destination over its whole [M, ldc] buffer; a tile lands at column col0 + n.  The 64-column
    // store boxes must not reach into the next rank's columns, hence N % 64 == 0 (checked by the caller).
    for (int d = 0; d < 8; ++d) {
      const uint64_t dims[3] = {(uint64_t)gd->ldc, (uint64_t)M, 1};
      const uint64_t str[2] = {(uint64_t)gd->ldc * 2, (uint64_t)M * (uint64_t)gd->ldc * 2};
      const uint32_t box[3] = {64, 32, 1};
      if (encode_map(&dst.m[d], CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, gd->dst[d < gd->n ? d : 0], dims, str, box,
                     CU_TENSOR_MAP_SWIZZLE_128B))
        return -1;
    }
  }
  qg::W8A8Params p;
  memset(&p, 0, sizeof(p));
  p.n_dst = gd ? gd->n : 0;
  p.col0 = gd ? (int)gd->col0 : 0;
  p.C = C;
  p.batch = (int)batch;
  p.M = (int)M;
  p.N = (int)N;
  p.K = (int)Kb;
  p.m_tiles = (int)m_tiles;
  p.group_m = w8_group_m(m_tiles, Kb);
  p.n_tiles = (int)((N + BN - 1) / BN);
  p.bn = BN;
  const int64_t num_tiles = batch * p.m_tiles * p.n_tiles;
  if (num_tiles > 0x7fffffff) return fail("qgemm_w4a16: too many tiles");
  p.num_tiles = (int)num_tiles;
  p.k_blocks = (int)((Kb + 127) / 128);
  p.status = status;
  p.wait_limit_ns = g_wait_limit_ns;
  p.tma_store = 1;
  p.split_from = p.num_items = p.num_tiles;
  const int grid = (int)(num_tiles < sms ? num_tiles : sms);
  if (BN == 256) {
    if (bf) qg::w8a8_gemm_kernel<256, true, true, true><<<grid, qg::W8_THREADS, qg::W8Cfg<256>::SMEM_BYTES, s>>>(tmA, tmB, dst, p);
    else qg::w8a8_gemm_kernel<256, true, false, true><<<grid, qg::W8_THREADS, qg::W8Cfg<256>::SMEM_BYTES, s>>>(tmA, tmB, dst, p);
  } else {
    if (bf) qg::w8a8_gemm_kernel<128, true, true, true><<<grid, qg::W8_THREADS, qg::W8Cfg<128>::SMEM_BYTES, s>>>(tmA, tmB, dst, p);
    else qg::w8a8_gemm_kernel<128, true, false, true><<<grid, qg::W8_THREADS, qg::W8Cfg<128>::SMEM_BYTES, s>>>(tmA, tmB, dst, p);
  }
  CUDA_OK(cudaGetLastError());
  return 0;
}

int qgemm_w4a16(const void* A, const uint8_t* B_packed, const void* scales, int zero, int64_t group, void* C,
                void* workspace, int64_t workspace_bytes, int64_t M, int64_t N, int64_t K, int a_dtype,
                int out_dtype, uint32_t* status, void* stream) {
  return qgemm_w4a16_batched(A, B_packed, scales, zero, group, C, workspace, workspace_bytes, 1, M, N, K, a_dtype,
                             out_dtype, status, stream);
}

static int w4a16_impl(const void* A, const uint8_t* B_packed, const void* scales, int zero, int64_t group, void* C,
                      void* workspace, int64_t workspace_bytes, int64_t batch, int64_t M, int64_t N, int64_t K,
                      int a_dtype, int out_dtype, uint32_t* status, void* stream, const void* zeros, int zero_mode,
                      int weight_format, const GatherDst* gd = nullptr);

int qgemm_w4a16_batched(const void* A, const uint8_t* B_packed, const void* scales, int zero, int64_t group, void* C,
                        void* workspace, int64_t workspace_bytes, int64_t batch, int64_t M, int64_t N, int64_t K,
                        int a_dtype, int out_dtype, uint32_t* status, void* stream) {
  return w4a16_impl(A, B_packed, scales, zero, group, C, workspace, workspace_bytes, batch, M, N, K, a_dtype, out_dtype,
                    status, stream, nullptr, QGEMM_ZERO_ORIGINAL, QGEMM_W4_SEQUENTIAL);
}

int qgemm_w4a16_ex(const void* A, const uint8_t* B_packed, const void* scales, const void* zeros, int zero,
                   int zero_mode, int weight_format, int64_t group, void* C, void* workspace, int64_t workspace_bytes,
                   int64_t batch, int64_t M, int64_t N, int64_t K, int a_dtype, int out_dtype, uint32_t* status,
                   void* stream) {
  if (weight_format != QGEMM_W4_SEQUENTIAL && weight_format != QGEMM_W4_INTERLEAVED_F16)
    return fail("qgemm_w4a16_ex: unknown weight_format %d", weight_format);
  if (zero_mode != QGEMM_ZERO_ORIGINAL && zero_mode != QGEMM_ZERO_RESCALE && zero_mode != QGEMM_ZERO_QUANTIZED)
    return fail("qgemm_w4a16_ex: unknown zero_mode %d", zero_mode);
  if (zeros == nullptr && zero_mode == QGEMM_ZERO_RESCALE)
    return fail("qgemm_w4a16_ex: zero mode 'rescale' needs the zeros tensor");
  if (zeros != nullptr) {
    if (scales == nullptr) return fail("qgemm_w4a16_ex: a zeros tensor needs scales");
    if (!aligned16(zeros)) return fail("qgemm_w4a16_ex: zeros must be 16-byte aligned");
    if (N % 16 != 0) return fail("qgemm_w4a16_ex: a zeros tensor needs N to be a multiple of 16 (got %lld)", (long long)N);
  }
  return w4a16_impl(A, B_packed, scales, zero, group, C, workspace, workspace_bytes, batch, M, N, K, a_dtype, out_dtype,
                    status, stream, zeros, zero_mode, weight_format);
}

static int w4a16_impl(const void* A, const uint8_t* B_packed, const void* scales, int zero, int64_t group, void* C,
                      void* workspace, int64_t workspace_bytes, int64_t batch, int64_t M, int64_t N, int64_t K,
                      int a_dtype, int out_dtype, uint32_t* status, void* stream, const void* zeros, int zero_mode,
                      int weight_format, const GatherDst* gd) {
  if (batch <= 0 || batch > 65535) return fail("qgemm_w4a16: batch must be in 1..65535 (got %lld)", (long long)batch);
  if (M <= 0 || N <= 0 || K <= 0) return fail("qgemm_w4a16: M, N, K must be positive (got %lld, %lld, %lld)", (long long)M, (long long)N, (long long)K);
  if (M > (1ll << 30) || N > (1ll << 30) || K > (1ll << 30)) return fail("qgemm_w4a16: dimension too large");
  if (A == nullptr || B_packed == nullptr || (C == nullptr && gd == nullptr)) return fail("qgemm_w4a16: A, B_packed and C must not be null");
  if (a_dtype != QGEMM_DT_F16 && a_dtype != QGEMM_DT_BF16) return fail("qgemm_w4a16: a_dtype must be F16 or BF16 (got %d)", a_dtype);
  if (out_dtype != QGEMM_DT_F16 && out_dtype != QGEMM_DT_BF16) return fail("qgemm_w4a16: out_dtype must be F16 or BF16 (got %d)", out_dtype);
  if (K % 32 != 0) return fail("qgemm_w4a16: K must be a multiple of 32 (got %lld)", (long long)K);
  if (N % 8 != 0) return fail("qgemm_w4a16: N must be a multiple of 8 (got %lld)", (long long)N);
  if (!aligned16(A) || !aligned16(B_packed) || !aligned16(C) || !aligned16(scales) || !aligned16(workspace)) return fail("qgemm_w4a16: pointers must be 16-byte aligned");
  if (scales != nullptr) {
    if (zero < 0 || zero > 15) return fail("qgemm_w4a16: zero must be in 0..15 (got %d)", zero);
    if (group <= 0 || K % group != 0) return fail("qgemm_w4a16: group must divide K (got group=%lld, K=%lld)", (long long)group, (long long)K);
    const bool ok = (group < 256 && 256 % group == 0 && group >= 32) || (group % 256 == 0) || (group >= K);
    if (!ok) return fail("qgemm_w4a16: group must be 32, 64, 128, a multiple of 256, or the whole K (got %lld)", (long long)group);
  } else {
    zero = 0;
    group = K;
  }
  // A zeros tensor of mode "quantized" (integer zero points) is taken in flight by the group-sum kernel wherever that
  // kernel applies; the other zero modes, whose f16 roundings per weight the group-sum form cannot reproduce, and all
  // other shapes go through the whole-matrix dequantisation.  QGEMM_W4_ZEROS_INFLIGHT=0 sends every zeros tensor there.
  static const int zeros_inflight_on = getenv("QGEMM_W4_ZEROS_INFLIGHT") ? atoi(getenv("QGEMM_W4_ZEROS_INFLIGHT")) : 1;
  const bool zeros_inflight = zeros != nullptr && zeros_inflight_on && zero_mode == QGEMM_ZERO_QUANTIZED && gd == nullptr &&
                              !w4_use_f16_gemm(M, N) && w4_gs_shape_ok(M, true, group, K);
  const bool dequant_once = (zeros != nullptr && !zeros_inflight) || w4_use_f16_gemm(M, N);
  // a zeros tensor that is taken in flight needs no room for dequantised weights
  const int64_t need = w4_workspace_bytes(batch, M, N, K, zeros != nullptr && !zeros_inflight);
  if (need < 0) return -1;
  if (workspace == nullptr || workspace_bytes < need) return fail("qgemm_w4a16: workspace of %lld bytes needed (got %lld)", (long long)need, (long long)workspace_bytes);

  int sms = 0;
  if (ensure_device(&sms)) return -1;
  const bool use_gs = !dequant_once && w4_gs_shape_ok(M, scales != nullptr, group, K);
  int mt = w4_pick_mt(M, use_gs);
  if (gd != nullptr && mt < 16) mt = 16;  // the register-operand decode kernel writes one destination only

  CUtensorMap tmW, tmS, tmZ, tmA;
  memset(&tmS, 0, sizeof(tmS));
  memset(&tmZ, 0, sizeof(tmZ));
  {
    const uint64_t dims[3] = {(uint64_t)(K / 2), (uint64_t)N, (uint64_t)batch};
    const uint64_t str[2] = {(uint64_t)(K / 2), (uint64_t)N * (uint64_t)(K / 2)};
    const uint32_t box[3] = {128, 128, 1};
    if (encode_map(&tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, B_packed, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
  }
  // the group-sum kernel fetches the scale rows of a slab's two 128-k halves: two rows for groups of 128, else one
  int scale_rows = 1;
  if (scales != nullptr) {
    scale_rows = use_gs ? (group == 128 ? 2 : 1) : (group < 256 ? (int)(256 / group) : 1);
    const uint64_t dims[3] = {(uint64_t)N, (uint64_t)(K / group), (uint64_t)batch};
    const uint64_t str[2] = {(uint64_t)N * 2, (uint64_t)(K / group) * (uint64_t)N * 2};
    const uint32_t box[3] = {128, (uint32_t)scale_rows, 1};
    if (encode_map(&tmS, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, scales, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE)) return -1;
    if (zeros_inflight &&
        encode_map(&tmZ, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, zeros, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE))
      return -1;
  }
  const int64_t grid_max = sms < kW4MaxGrid ? sms : kW4MaxGrid;
  uint8_t* a_prepared = static_cast<uint8_t*>(workspace) + kW4CounterBytes + grid_max * 2 * (int64_t)mt * 128 * 4;
  {
    const uint64_t dims[3] = {(uint64_t)K, (uint64_t)M, (uint64_t)batch};
    const uint64_t str[2] = {(uint64_t)K * 2, (uint64_t)M * (uint64_t)K * 2};
    const uint32_t box[3] = {64, (uint32_t)mt, 1};
    if (encode_map(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, a_prepared, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
  }

  qg::W4A16Params p;
  p.C = C;
  p.n_dst = 0;
  p.ldc = p.col0 = 0;
  for (int d = 0; d < 8; ++d) p.c_dst[d] = nullptr;
  if (gd != nullptr) {
    p.n_dst = gd->n;
    p.ldc = (int)gd->ldc;
    p.col0 = (int)gd->col0;
    for (int d = 0; d < gd->n; ++d) p.c_dst[d] = gd->dst[d];
  }
  p.ws_counters = static_cast<uint32_t*>(workspace);
  p.ws_partials = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + kW4CounterBytes);
  p.M = (int)M;
  p.N = (int)N;
  p.K = (int)K;
  p.group = (int)(group > (1 << 30) ? (1 << 30) : group);
  p.zero = zero;
  p.has_scales = scales != nullptr;
  p.m_tiles = (int)((M + mt - 1) / mt);
  p.n_tiles = (int)((N + 127) / 128);
  p.batch = (int)batch;
  const int64_t num_tiles = batch * (int64_t)p.m_tiles * p.n_tiles;
  if (num_tiles > 0x3fffffff) return fail("qgemm_w4a16: too many tiles");
  p.num_tiles = (int)num_tiles;
  p.KS = (int)((K + 255) / 256);
  p.scale_rows = scale_rows;
  p.total_items = num_tiles * p.KS;
  p.status = status;
  p.wait_limit_ns = g_wait_limit_ns;
  p.A_raw = nullptr;
  p.a_is_bf16 = p.a_permute = 0;
  int64_t grid = sms < kW4MaxGrid ? sms : kW4MaxGrid;
  if (p.total_items < grid) grid = p.total_items;
  // Small problems (a few slabs per CTA): prefer a slightly smaller grid that cuts every tile into equal K ranges,
  // one per CTA, over an even deal that leaves most CTAs with two partial tiles and so two split-K hand-overs.
  if (p.total_items <= 8 * grid && p.total_items > grid) {
    for (int64_t g2 = grid; g2 * 4 >= grid * 3; --g2) {
      if (p.total_items % g2 != 0) continue;
      const int64_t per = p.total_items / g2;
      if (p.KS % per == 0) {
        grid = g2;
        break;
      }
    }
  }
  // Group-sum kernel, 16-token tile: whole tiles per CTA where there are enough, and only the remainder (plus one
  // round when the remainder alone would give every CTA a sliver of a tile) cut stream-K fashion, processed first, so
  // that the launch ends with plain tile writes instead of the partial tiles' hand-overs (K=8192, N=28672: 38.2 ->
  // 36.5 us at 16 tokens, 37.7 -> 36.1 at 8).  The taller tiles keep the even cut: their drain warps set the pace,
  // and a hand-over in the middle of a CTA's work stalls them where one at the end only delays the exit (measured
  // 4 % slower at 32 tokens, 3 % at 64).  QGEMM_W4_HYBRID=0 cuts all tiles stream-K fashion.
  p.sk_tiles = p.num_tiles;
  p.dp_rounds = 0;
  {
    static const int hybrid = getenv("QGEMM_W4_HYBRID") ? atoi(getenv("QGEMM_W4_HYBRID")) : 1;
    const int64_t rounds = num_tiles / grid, r = num_tiles % grid;
    if (hybrid && use_gs && mt == 16 && rounds >= 1) {
      const bool borrow = r != 0 && 2 * r < grid;
      p.dp_rounds = (int)(borrow ? rounds - 1 : rounds);
      p.sk_tiles = (int)(borrow ? r + grid : r);
    }
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool bf = out_dtype == QGEMM_DT_BF16;
  // Problems of a few slabs per CTA (16 tokens at most, K <= 4096: every tile's K cut over a cluster of 1, 2 or 4 CTAs
  // with at most four slabs each, all clusters resident at once): one launch, no pre-pass, no scratch - see the
  // kernel's SMALL parameter.  Measured against the two-launch form: 16 x 4096 x 4096 9.2 / 10.6 us, 16 x 2048 x 8192
  // 8.8 / 9.8 us; with more clusters than SMs (several waves) it loses.  QGEMM_W4_SMALL=0 keeps the two-launch form.
  {
    static const int small_on = getenv("QGEMM_W4_SMALL") ? atoi(getenv("QGEMM_W4_SMALL")) : 1;
    if (small_on && use_gs && mt == 16 && gd == nullptr && !zeros_inflight && g_w4g_withhold_commit != 1) {
      int cluster = 0;
      for (int c = 1; c <= 4; c *= 2)  // clusters of eight were measured slower than the two-launch form (15.3 / 11.3 us)
        if (p.KS % c == 0 && p.KS / c <= qg::W4G_SMALL_MAX_SLABS) { cluster = c; break; }
      static const int small_waves = getenv("QGEMM_W4_SMALL_WAVES") ? atoi(getenv("QGEMM_W4_SMALL_WAVES")) : 1;
      if (cluster > 0 && num_tiles * cluster <= (int64_t)small_waves * sms) {
        p.A_raw = A;
        p.a_is_bf16 = a_dtype == QGEMM_DT_BF16 ? 1 : 0;
        p.a_permute = weight_format == QGEMM_W4_SEQUENTIAL ? 1 : 0;
        return launch_w4g_small(bf, tmW, tmS, tmA, p, (int)(num_tiles * cluster), cluster, s);
      }
    }
  }
  {
    const long long n_chunks = (long long)batch * M * K / 8;
    const long long blocks = (n_chunks + 255) / 256;
    if (blocks > 0x7fffffffll) return fail("qgemm_w4a16: activation tensor too large");
    // Launched as a programmatic dependent too: behind another call of this operator (whose GEMM kernel lets its
    // dependents go at once) the pre-pass is already resident, waiting, when that call ends, and the GEMM kernel
    // behind it sets up and streams its first weights meanwhile.  Behind any other kernel this is plain stream order.
    const uint4* a_in = static_cast<const uint4*>(A);
    uint4* a_out = reinterpret_cast<uint4*>(a_prepared);
    const int is_bf = a_dtype == QGEMM_DT_BF16 ? 1 : 0, permute = weight_format == QGEMM_W4_SEQUENTIAL ? 1 : 0;
    if (launch_pdl(qg::w4a16_prepare_activations, (int)blocks, 256, 0, s, a_in, a_out, n_chunks, is_bf, permute,
                   p.ws_counters, (int)(kW4CounterBytes / 4)))
      return -1;
  }
  if (dequant_once) {
    uint8_t* w16 = a_prepared + batch * M * K * 2;
    const int64_t geff = group > K ? K : group;
    const long long n_chunks = (long long)batch * N * (K / 32);
    const long long blocks = (n_chunks + 255) / 256;
    if (blocks > 0x7fffffffll) return fail("qgemm_w4a16: weight tensor too large");
    qg::w4a16_dequant_weights<<<(unsigned)blocks, 256, 0, s>>>(reinterpret_cast<const uint4*>(B_packed),
                                                             static_cast<const __half*>(scales),
                                                             static_cast<const __half*>(zeros), zero_mode,
                                                             reinterpret_cast<uint4*>(w16), n_chunks, (int)(K / 32),
                                                             (int)N, (int)K, (int)geff, zero);
    CUDA_OK(cudaGetLastError());
    return w4_f16_gemm(a_prepared, w16, C, batch, M, N, K, bf, status, s, sms, gd);
  }
  if (use_gs) {
    const CUtensorMap* tz = zeros_inflight ? &tmZ : nullptr;
    if (mt == 16) return launch_w4g<16>(bf, tmW, tmS, tz, tmA, p, (int)grid, s);
    if (mt == 32) return launch_w4g<32>(bf, tmW, tmS, tz, tmA, p, (int)grid, s);
    return launch_w4g<64>(bf, tmW, tmS, tz, tmA, p, (int)grid, s);
  }
  if (gd == nullptr && w4_use_decode(M) && mt <= 16 && M <= w4_decode_max_m()) {
    if (scales == nullptr) return launch_w4d<0>(bf, mt, tmW, tmS, tmA, p, (int)grid, s);
    if (group >= 128) return launch_w4d<4>(bf, mt, tmW, tmS, tmA, p, (int)grid, s);
    if (group == 64) return launch_w4d<2>(bf, mt, tmW, tmS, tmA, p, (int)grid, s);
    return launch_w4d<1>(bf, mt, tmW, tmS, tmA, p, (int)grid, s);
  }
  switch (mt) {
    case 16: return launch_w4<16>(bf, tmW, tmS, tmA, p, (int)grid, s);
    case 32: return launch_w4<32>(bf, tmW, tmS, tmA, p, (int)grid, s);
    case 64: return launch_w4<64>(bf, tmW, tmS, tmA, p, (int)grid, s);
    default: return launch_w4<128>(bf, tmW, tmS, tmA, p, (int)grid, s);
  }
}

int qgemm_w4a16_gather(const void* A, const uint8_t* B_packed, const void* scales, int zero, int64_t group,
                       void* const* C_dst, int n_dst, int64_t ldc, int64_t col0, void* workspace,
                       int64_t workspace_bytes, int64_t M, int64_t N, int64_t K, int a_dtype, int out_dtype,
                       uint32_t* status, void* stream) {
  if (C_dst == nullptr || n_dst < 1 || n_dst > 8) return fail("qgemm_w4a16_gather: 1 to 8 destinations required (got %d)", n_dst);
  for (int d = 0; d < n_dst; ++d)
    if (C_dst[d] == nullptr || !aligned16(C_dst[d])) return fail("qgemm_w4a16_gather: destination %d is null or not 16-byte aligned", d);
  if (ldc <= 0 || ldc > (1ll << 30) || col0 < 0 || N <= 0 || col0 + N > ldc)
    return fail("qgemm_w4a16_gather: columns [%lld, %lld) do not fit in rows of %lld", (long long)col0, (long long)(col0 + N), (long long)ldc);
  if (ldc % 8 != 0 || col0 % 8 != 0) return fail("qgemm_w4a16_gather: ldc and col0 must be multiples of 8 (got %lld, %lld)", (long long)ldc, (long long)col0);
  if (w4_use_f16_gemm(M, N) && N % 64 != 0)
    return fail("qgemm_w4a16_gather: from %lld tokens on N must be a multiple of 64 (got %lld)", (long long)w4_gemm_min_m(), (long long)N);
  GatherDst gd{C_dst, n_dst, ldc, col0};
  return w4a16_impl(A, B_packed, scales, zero, group, nullptr, workspace, workspace_bytes, 1, M, N, K, a_dtype, out_dtype,
                    status, stream, nullptr, QGEMM_ZERO_ORIGINAL, QGEMM_W4_SEQUENTIAL, &gd);
}

}  // extern "C"

// ---- "my blocks have landed" between the ranks of the gathered form ----
namespace {
struct PeerSlots {
  uint32_t* slot[8];
};
// Thread r: release-store the epoch into this rank's slot of rank r's flag array, then acquire-poll slot r of this
// rank's own array until rank r's epoch has arrived.  Bounded: gives up after limit_ns and reports it.
__global__ void peer_signal_wait_kernel(PeerSlots dst, const uint32_t* local_flags, int n, uint32_t epoch,
                                        uint32_t* epoch_counter, unsigned long long limit_ns, uint32_t* status) {
  __shared__ uint32_t epoch_s;
  const int r = threadIdx.x;
  if (epoch_counter != nullptr) {  // the epoch lives on the device: replays of a captured launch keep counting
    if (r == 0) {
      epoch_s = *epoch_counter + 1u;
      *epoch_counter = epoch_s;
    }
    __syncthreads();
    epoch = epoch_s;
  }
  if (r >= n) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst.slot[r]), "r"(epoch) : "memory");
  const uint32_t* mine = local_flags + r;
  const unsigned long long t0 = qg::global_timer_ns();
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if ((int32_t)(v - epoch) >= 0) break;
    if (qg::global_timer_ns() - t0 > limit_ns) {
      if (status != nullptr) atomicMax(status, (uint32_t)qg::ST_TIMEOUT_PEER);
      break;
    }
    __nanosleep(100);
  }
}
}  // namespace

extern "C" {

int qgemm_peer_signal_wait(void* const* flag_slots, int n, const uint32_t* local_flags, uint32_t epoch,
                           uint32_t* epoch_counter, uint32_t* status, void* stream) {
  if (flag_slots == nullptr || local_flags == nullptr || n < 1 || n > 8) return fail("qgemm_peer_signal_wait: 1 to 8 ranks, non-null flag arrays required (got n=%d)", n);
  PeerSlots dst;
  for (int r = 0; r < 8; ++r) dst.slot[r] = nullptr;
  for (int r = 0; r < n; ++r) {
    if (flag_slots[r] == nullptr || (reinterpret_cast<uintptr_t>(flag_slots[r]) & 3u) != 0) return fail("qgemm_peer_signal_wait: flag slot %d is null or misaligned", r);
    dst.slot[r] = static_cast<uint32_t*>(flag_slots[r]);
  }
  peer_signal_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(dst, local_flags, n, epoch, epoch_counter, g_wait_limit_ns, status);
  CUDA_OK(cudaGetLastError());
  return 0;
}

// ---- mapping another process's buffer into this one (same node), for the gathered form ----
static_assert(sizeof(cudaIpcMemHandle_t) == QGEMM_IPC_HANDLE_BYTES, "IPC handle size");

int qgemm_ipc_export(const void* dev_ptr, void* handle_out, int64_t* offset_out) {
  if (dev_ptr == nullptr || handle_out == nullptr || offset_out == nullptr) return fail("qgemm_ipc_export: null argument");
  int sms = 0;
  if (ensure_device(&sms)) return -1;
  // the handle names the whole allocation the pointer lies in; the pointer's offset inside it travels with it
  using RangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
  static RangeFn range_fn = nullptr;
  if (range_fn == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    CUDA_OK(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qres));
    if (qres != cudaDriverEntryPointSuccess || fn == nullptr) return fail("cuMemGetAddressRange not available from the driver");
    range_fn = reinterpret_cast<RangeFn>(fn);
  }
  CUdeviceptr base = 0;
  size_t size = 0;
  const CUresult r = range_fn(&base, &size, reinterpret_cast<CUdeviceptr>(dev_ptr));
  if (r != CUDA_SUCCESS) return fail("cuMemGetAddressRange failed with CUresult %d", (int)r);
  cudaIpcMemHandle_t h;
  CUDA_OK(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
  memcpy(handle_out, &h, sizeof(h));
  *offset_out = (int64_t)(reinterpret_cast<CUdeviceptr>(dev_ptr) - base);
  return 0;
}

int qgemm_ipc_open(const void* handle, void** base_out) {
  if (handle == nullptr || base_out == nullptr) return fail("qgemm_ipc_open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* ptr = nullptr;
  CUDA_OK(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
  *base_out = ptr;
  return 0;
}

int qgemm_ipc_close(void* base) {
  if (base == nullptr) return 0;
  CUDA_OK(cudaIpcCloseMemHandle(base));
  return 0;
}

int qgemm_unpack_int4(const uint8_t* B_packed, int8_t* out, int64_t N, int64_t K, int signed_nibbles,
                      void* stream) {
  if (N <= 0 || K <= 0 || (K % 2) != 0) return fail("qgemm_unpack_int4: N, K must be positive and K even (got %lld, %lld)", (long long)N, (long long)K);
  if (B_packed == nullptr || out == nullptr) return fail("qgemm_unpack_int4: null pointer");
  if (!aligned16(B_packed) || !aligned16(out)) return fail("qgemm_unpack_int4: pointers must be 16-byte aligned");
  const long long n_bytes = (long long)N * (K / 2);
  const long long threads = (n_bytes + 15) / 16;
  const int block = 256;
  const long long grid = (threads + block - 1) / block;
  if (grid > 0x7fffffffll) return fail("qgemm_unpack_int4: tensor too large");
  unpack_int4_kernel<<<(unsigned)grid, block, 0, static_cast<cudaStream_t>(stream)>>>(B_packed, out, n_bytes, signed_nibbles);
  CUDA_OK(cudaGetLastError());
  return 0;
}

int qgemm_act_quant(const void* X, int8_t* Y, float* S, int64_t M, int64_t N, int x_dtype, int round_scale,
                    void* stream) {
  if (M < 0 || N <= 0 || (N % 8) != 0) return fail("qgemm_act_quant: M >= 0 and N a positive multiple of 8 required (got M=%lld, N=%lld)", (long long)M, (long long)N);
  if (N > (1ll << 30)) return fail("qgemm_act_quant: N too large (%lld)", (long long)N);
  if (x_dtype != QGEMM_DT_F16 && x_dtype != QGEMM_DT_BF16) return fail("qgemm_act_quant: x_dtype must be F16 or BF16 (got %d)", x_dtype);
  if (M == 0) return 0;
  if (X == nullptr || Y == nullptr || S == nullptr) return fail("qgemm_act_quant: null pointer");
  if (!aligned16(X) || (reinterpret_cast<uintptr_t>(Y) & 7u) != 0 || (reinterpret_cast<uintptr_t>(S) & 3u) != 0)
    return fail("qgemm_act_quant: X must be 16-byte, Y 8-byte and S 4-byte aligned");
  qg::ActQuantParams p;
  p.X = static_cast<const uint4*>(X);
  p.Y = Y;
  p.S = S;
  p.M = M;
  p.N = (int)N;
  p.is_bf16 = x_dtype == QGEMM_DT_BF16;
  p.round_scale = round_scale != 0;
  const int64_t chunks = N / 8;
  // threads per row: the fewest of 32..256 that keep a row in at most 4 chunks per thread (8 at 256)
  int tpr = 32;
  while (tpr < qg::AQ_THREADS && chunks > (int64_t)tpr * 4) tpr *= 2;
  const bool keep8 = chunks > (int64_t)tpr * 4;
  const int64_t rows_per_block = qg::AQ_THREADS / tpr;
  const int64_t grid = (M + rows_per_block - 1) / rows_per_block;
  if (grid > 0x7fffffffll) return fail("qgemm_act_quant: too many rows (%lld)", (long long)M);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (tpr) {
    case 32: qg::act_quant_kernel<32, 4><<<(unsigned)grid, qg::AQ_THREADS, 0, st>>>(p); break;
    case 64: qg::act_quant_kernel<64, 4><<<(unsigned)grid, qg::AQ_THREADS, 0, st>>>(p); break;
    case 128: qg::act_quant_kernel<128, 4><<<(unsigned)grid, qg::AQ_THREADS, 0, st>>>(p); break;
    default:
      if (keep8) qg::act_quant_kernel<256, qg::AQ_MAX_CHUNKS><<<(unsigned)grid, qg::AQ_THREADS, 0, st>>>(p);
      else qg::act_quant_kernel<256, 4><<<(unsigned)grid, qg::AQ_THREADS, 0, st>>>(p);
      break;
  }
  CUDA_OK(cudaGetLastError());
  return 0;
}

int qgemm_w4a8(const int8_t* A, const uint8_t* qB, int8_t* workspace, void* C, int64_t M, int64_t N, int64_t K,
               int signed_nibbles, int out_dtype, uint32_t* status, void* stream) {
  if (workspace == nullptr) return fail("qgemm_w4a8: the int8 [N, K] workspace must not be null");
  if (K % 32 != 0 || N % 16 != 0) return fail("qgemm_w4a8: K must be a multiple of 32 and N of 16 (got K=%lld, N=%lld)", (long long)K, (long long)N);
  if (out_dtype == QGEMM_DT_I32 && M > 0 && N > 0 && K > 0 && A != nullptr && qB != nullptr && C != nullptr &&
      aligned16(A) && aligned16(qB) && aligned16(C)) {
    const int rc = w4a8_fused(A, qB, workspace, static_cast<int*>(C), M, N, K, signed_nibbles, status,
                              static_cast<cudaStream_t>(stream));
    if (rc <= 0) return rc;
  }
  if (qgemm_unpack_int4(qB, workspace, N, K, signed_nibbles, stream)) return -1;
  if (out_dtype == QGEMM_DT_I32)
    return qgemm_w8a8(A, workspace, nullptr, nullptr, C, nullptr, 1, M, N, K, 1, 0, QGEMM_DT_I32, QGEMM_B_NK, status, stream);
  return fail("qgemm_w4a8: out_dtype must be I32; cast the result on the caller's side (got %d)", out_dtype);
}

int qgemm_w4a8_act_quant(const void* X, int x_dtype, const uint8_t* qB, int8_t* workspace, int32_t* C, float* scale_a,
                         int round_scale, int64_t M, int64_t N, int64_t K, int signed_nibbles, uint32_t* status,
                         void* stream) {
  if (X == nullptr || qB == nullptr || workspace == nullptr || C == nullptr || scale_a == nullptr)
    return fail("qgemm_w4a8_act_quant: X, qB, workspace, C and scale_a must not be null");
  if (x_dtype != QGEMM_DT_F16 && x_dtype != QGEMM_DT_BF16) return fail("qgemm_w4a8_act_quant: x_dtype must be F16 or BF16 (got %d)", x_dtype);
  if (M <= 0 || N <= 0 || K <= 0) return fail("qgemm_w4a8_act_quant: M, N, K must be positive (got %lld, %lld, %lld)", (long long)M, (long long)N, (long long)K);
  if (K % 32 != 0 || N % 16 != 0) return fail("qgemm_w4a8_act_quant: K must be a multiple of 32 and N of 16 (got K=%lld, N=%lld)", (long long)K, (long long)N);
  if (!aligned16(X) || !aligned16(qB) || !aligned16(C) || !aligned16(workspace)) return fail("qgemm_w4a8_act_quant: pointers must be 16-byte aligned");
  if (M > 128)
    return fail("qgemm_w4a8_act_quant: the fused form covers M <= 128 (got %lld); use qgemm_act_quant and qgemm_w4a8 above that", (long long)M);
  const int rc = w4a8_fused(nullptr, qB, workspace, C, M, N, K, signed_nibbles, status, static_cast<cudaStream_t>(stream), X,
                            x_dtype == QGEMM_DT_BF16 ? 1 : 0, round_scale, scale_a);
  if (rc > 0) return fail("qgemm_w4a8_act_quant: the [N, K] workspace is too small for the kernel's scratch (N * K = %lld bytes)", (long long)(N * K));
  return rc;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------
// Allocation-free W4A16 entry point.
//
// The scratch memory of the W4A16 kernels (split-K arrival counters, fp32 partial sums, the f16 copy
// of the activations) lives here in a device array that is part of the library image, so a caller
// never has to provide or allocate it.  Every GPU that loads the library carries this array until the
// process exits.
// ---------------------------------------------------------------------------------------------------
namespace {

constexpr int64_t kStaticMaxM = QGEMM_W4A16_NOALLOC_MAX_M;
constexpr int64_t kStaticMaxK = QGEMM_W4A16_NOALLOC_MAX_K;
constexpr int64_t kStaticMaxSms = 160;
constexpr int64_t kStaticScratchBytes =
    kW4CounterBytes + kStaticMaxSms * 2 * kStaticMaxM * 128 * 4 + kStaticMaxM * kStaticMaxK * 2;  // about 6.3 MB

static __device__ __align__(256) unsigned char g_w4a16_static_scratch[kStaticScratchBytes];

// Device address of the array above, per device.  In host code the array's name is only a handle for
// the runtime, not a pointer a kernel could use: the real address comes from cudaGetSymbolAddress and
// differs from GPU to GPU.
void* g_static_scratch_addr[kMaxDevices] = {};
std::mutex g_static_mu;

int static_scratch_for_current_device(void** out) {
  int dev = 0;
  CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail("device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (g_static_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    CUDA_OK(cudaGetSymbolAddress(&ptr, g_w4a16_static_scratch));
    if (ptr == nullptr) return fail("cudaGetSymbolAddress returned a null address for the static scratch array");
    g_static_scratch_addr[dev] = ptr;
  }
  *out = g_static_scratch_addr[dev];
  return 0;
}

}  // namespace

extern "C" int qgemm_w4a16_noalloc(const void* A, const uint8_t* B_packed, const void* scales, int zero,
                                   int64_t group, void* C, int64_t M, int64_t N, int64_t K, int a_dtype,
                                   int out_dtype, uint32_t* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return fail("qgemm_w4a16_noalloc: M, N, K must be positive (got %lld, %lld, %lld)", (long long)M, (long long)N, (long long)K);
  if (M > kStaticMaxM || K > kStaticMaxK)
    return fail("qgemm_w4a16_noalloc: the built-in scratch covers M <= %lld and K <= %lld (got M=%lld, K=%lld); "
                "use qgemm_w4a16 with a caller-provided workspace for larger problems",
                (long long)kStaticMaxM, (long long)kStaticMaxK, (long long)M, (long long)K);
  const int64_t need = qgemm_w4a16_workspace_bytes(M, N, K);
  if (need < 0) return -1;
  if (need > kStaticScratchBytes)
    return fail("qgemm_w4a16_noalloc: this problem needs %lld bytes of scratch on this device, the built-in array has %lld",
                (long long)need, (long long)kStaticScratchBytes);
  void* scratch = nullptr;
  if (static_scratch_for_current_device(&scratch)) return -1;
  // The array keeps whatever the previous call left behind.  The arrival counters must start at zero: the
  // pre-pass kernel of every call zeroes them; everything else is written before it is read.  Nothing is put
  // on the stream before qgemm_w4a16 has validated the remaining arguments.
  return qgemm_w4a16(A, B_packed, scales, zero, group, C, scratch, kStaticScratchBytes, M, N, K, a_dtype, out_dtype,
                     status, stream);
}
