/*
 * qgemm.h — C ABI of libqgemm.so: quantized GEMM operators for NVIDIA B200 (sm_100a).
 *
 * This is the drop-in boundary for the quantized-GEMM operators of tile-ai/tilelang-ascend
 * (examples/quant_batch_matmul, examples/dequantize_gemm, packing as in tilelang/quantize).
 * In the reference every compiled operator is a shared object that exports
 *     extern "C" void call(uint8_t* arg0, ..., <int64 dynamic dims>, aclrtStream stream)
 * (src/target/codegen_ascend.cc:1061-1112), called through ctypes with raw device pointers in
 * parameter order, outputs and workspaces included, stream last
 * (tilelang/jit/adapter/cython/cython_wrapper.pyx:143-197).  The entry points below keep that
 * convention — plain device pointers, sizes as int64, stream last, asynchronous launch, no host
 * synchronisation — and add what the reference's CUDA-flavoured wrapper template defines and its
 * NPU build leaves out (tilelang/jit/adapter/wrapper.py:30-50): an init call, an int return code
 * and a last-error string.
 *
 * Rules common to all entry points
 *  - All pointers are device pointers on the current CUDA device, tensors are contiguous row-major.
 *  - Nothing is allocated or freed on the device and no pointer is retained after return.
 *  - Return value 0 = launched; non-zero = rejected before any launch, qgemm_last_error() says why.
 *  - `status` (nullable) is a device uint32 the caller zeroes; a kernel whose bounded wait expired
 *    stores a non-zero code there (see QGEMM_ST_*), drains and returns normally.
 *  - `stream` is a cudaStream_t passed as void* (NULL = default stream).
 */
#ifndef QGEMM_H_
#define QGEMM_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QGEMM_DT_F16 0
#define QGEMM_DT_BF16 1
#define QGEMM_DT_I32 2

#define QGEMM_B_KN 0 /* B stored [batch, K, N], N contiguous (examples/quant_batch_matmul) */
#define QGEMM_B_NK 1 /* B stored [batch, N, K], K contiguous (examples/deepseek_v4/int8_gemm.py:58) */

#define QGEMM_ST_OK 0
#define QGEMM_ST_TIMEOUT_PRODUCER 1
#define QGEMM_ST_TIMEOUT_MMA 2
#define QGEMM_ST_TIMEOUT_EPILOGUE 3
#define QGEMM_ST_TIMEOUT_DEQUANT 4
#define QGEMM_ST_TIMEOUT_DRAIN 5
#define QGEMM_ST_TIMEOUT_PEER 6      /* qgemm_peer_signal_wait: a peer's signal did not arrive within the wait limit */

/* Library version (major * 1000 + minor). */
int qgemm_version(void);

/* Per-device set-up (kernel attributes, driver entry points) for the current device.  Optional:
 * every entry point does it on first use.  Replaces `int init()` of
 * tilelang/jit/adapter/wrapper.py:36-43. */
int qgemm_init(void);

/* Message of the last non-zero return on the calling thread.  Replaces `get_last_error()` of
 * tilelang/jit/adapter/wrapper.py:30-34. */
const char* qgemm_last_error(void);

/* Per-wait limit of the kernels' bounded waits, in milliseconds (default 2000). */
void qgemm_set_wait_limit_ms(uint32_t ms);

/* Test hook, off by default (no counterpart in the reference).  With 1 the small-token W4A16 kernel (two-launch
 * form) leaves one accumulator hand-over of the launch unsignalled; with 2 the single-launch form of small problems
 * keeps back one CTA's "my sums have arrived" signal inside the last cluster.  Either way one bounded wait of the
 * epilogue runs out: the launch ends after the wait limit with QGEMM_ST_TIMEOUT_EPILOGUE in `status` and an
 * unspecified C, nothing is left in flight and the next call works normally.  It exists so that a test can see the
 * time-out paths end to end without faulting or hanging the device. */
void qgemm_debug_withhold_commit(int on);

/*
 * W8A8 quantized (batched) matmul.  Replaces the compiled `call` of
 * simple_quant_batch_matmul / simple_quant_matmul
 * (examples/quant_batch_matmul/example_quant_batch_matmul.py:17-91, example_quant_matmul.py:17-90)
 * and of the two-scale kernel examples/deepseek_v4/int8_gemm.py:35-104.
 *
 *   acc[b,m,n] = sum_k int32(A[b,m,k]) * int32(B[b,k,n])                          (exact)
 *   C[b,m,n]   = cast_out( float(acc) [* scale_a[..m]] * scale_b[..n] )            (fp32, RN casts)
 *
 * A: [batch, M, K] int8.  B: [batch, K, N] (QGEMM_B_KN) or [batch, N, K] (QGEMM_B_NK) int8.
 * scale_b: fp32, scale_b_len = 1, N (shared by all batches) or batch*N.
 * scale_a: nullable fp32, scale_a_len = 0, M (shared) or batch*M.
 * C: [batch, M, N] of out_dtype (F16 / BF16), or NULL when only accumulators are wanted; with
 *    out_dtype = QGEMM_DT_I32, C receives the raw int32 accumulators and the scales are ignored.
 * acc_out: nullable [batch, M, N] int32 — the reference's `workspace_1` (example_quant_batch_matmul.py:42),
 *    filled with the raw accumulators when given.
 * Unbatched operators pass batch = 1.  Requires K % 16 == 0 and N % 16 == 0.
 */
int qgemm_w8a8(const int8_t* A, const int8_t* B, const float* scale_b, const float* scale_a, void* C,
               int32_t* acc_out, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t scale_b_len,
               int64_t scale_a_len, int out_dtype, int b_layout, uint32_t* status, void* stream);

/*
 * Grouped (ragged) W8A8 matmul: row groups of different sizes, stacked in one A, each multiplied by its own
 * B.  The quantized counterpart of the grouped GEMM of examples/grouped_gemm/example_grouped_gemm_fwd.py:44-113
 * (same operands and the same host-built table; the int8 arithmetic and the scale epilogue are qgemm_w8a8's).
 *
 *   for every row block i = (g, m0, rows) of block_metadata and r < rows:
 *     acc[m0+r, n] = sum_k int32(A[m0+r, k]) * int32(B[g, k, n])
 *     C[m0+r, n]   = cast_out( float(acc) [* scale_a[m0+r]] * scale_b[g or 0, n] )
 *
 * A: [total_M, K] int8.  B: [groups, K, N] (QGEMM_B_KN) or [groups, N, K] (QGEMM_B_NK) int8.
 * block_metadata: device int32 [num_blocks, 3] = (group index, first row in A / C, valid rows), as
 *    construct_inputs builds it (example_grouped_gemm_fwd.py:147-166), with at most 128 rows per block.
 *    Unlike the reference kernel (README.md:16-22) partial blocks are allowed: only `rows` rows are written.
 *    Rows of C that no block covers are left untouched.  An entry that points outside the tensors is skipped.
 * scale_b: fp32, scale_b_len = 1, N or groups*N.  scale_a: nullable fp32 [total_M].  C, acc_out, out_dtype,
 * b_layout, status, stream as qgemm_w8a8.  Requires K % 16 == 0 and N % 16 == 0.
 */
int qgemm_w8a8_grouped(const int8_t* A, const int8_t* B, const float* scale_b, const float* scale_a, void* C,
                       int32_t* acc_out, const int32_t* block_metadata, int64_t num_blocks, int64_t groups,
                       int64_t total_M, int64_t N, int64_t K, int64_t scale_b_len, int64_t scale_a_len, int out_dtype,
                       int b_layout, uint32_t* status, void* stream);

/* Bytes of scratch memory qgemm_w4a16 needs for this problem on the current device (split-K partial
 * sums and arrival counters, the prepared activations and, from 1792 tokens on, the weights as f16: 2*N*K).
 * The buffer needs no initialisation: every call zeroes the qgemm_w4a16_counter_bytes() bytes of arrival
 * counters at its start, on the stream, and writes everything else before reading it.  Two launches
 * that may overlap on the device must not share a scratch buffer. */
int64_t qgemm_w4a16_workspace_bytes(int64_t M, int64_t N, int64_t K);
int64_t qgemm_w4a16_counter_bytes(void);

/*
 * W4A16 dequantize-GEMM.  Replaces dequant_gemm_fp16_wrapper's host unpack + compiled fp16 GEMM
 * (examples/dequantize_gemm/example_dequant_gemm_fine_grained.py:69-115,176-223); the scaled form
 * follows tilelang/quantize/utils.py:33,46 and zero mode "original" of tilelang/quantize/lop3.py:135-175.
 *
 *   q[n,k]  = (B_packed[n, k/2] >> 4*(k%2)) & 0xF            (low nibble = even k)
 *   W[n,k]  = scales ? half(q - zero) * scales[k/group, n] : half(q)
 *   C[m,n]  = cast_out( sum_k float(A[m,k]) * float(W[n,k]) )   (fp32 accumulation)
 *
 * Where the scale enters depends on the token count.  Up to 64 tokens (groups of 128, multiples of 256 or
 * the whole K) the kernels keep (q - zero) exact in f16, accumulate each group in fp32 and multiply the
 * group's sum by its scale in fp32: C = cast_out( sum_g scales[g,n] * sum_{k in g} A[m,k] * (q - zero) ).
 * Above that (and for groups of 32 / 64) every weight is scaled in f16 first, W rounded once as written
 * above.  Both forms give the same result bit for bit when a row of A is one-hot, and differ otherwise by
 * at most the rounding of that f16 product, 2^-11 relative per term; both meet rtol = atol = 1e-2 against
 * the fp32 reference program.  The same inputs may therefore differ in the last bits between, say, M = 64
 * and M = 65.
 *
 * A: [M, K] of a_dtype (F16 / BF16; bf16 is converted to f16 on the fly, as the reference wrapper does,
 *    example_dequant_gemm_fine_grained.py:211-214).  B_packed: [N, K/2] uint8.
 * scales: nullable [K/group, N] fp16; with scales == NULL `zero` and `group` are ignored.
 * C: [M, N] of out_dtype (F16 / BF16).  workspace: scratch of at least qgemm_w4a16_workspace_bytes().
 * Requires K % 32 == 0, N % 8 == 0, 0 <= zero <= 15, and group dividing 256, a multiple of 256, or >= K
 * (with K % group == 0).
 */
int qgemm_w4a16(const void* A, const uint8_t* B_packed, const void* scales, int zero, int64_t group, void* C,
                void* workspace, int64_t workspace_bytes, int64_t M, int64_t N, int64_t K, int a_dtype,
                int out_dtype, uint32_t* status, void* stream);

/*
 * Batched W4A16: `batch` independent problems of one shape in a single launch (for example the experts of
 * a mixture layer, or several projections applied to their own activations), the W4A16 analogue of the
 * batch dimension of simple_quant_batch_matmul (examples/quant_batch_matmul/example_quant_batch_matmul.py:38-41).
 * A: [batch, M, K]; B_packed: [batch, N, K/2]; scales: nullable [batch, K/group, N]; C: [batch, M, N];
 * everything else as qgemm_w4a16, which is the batch = 1 case.  All (problem, tile, K slab) work items
 * are dealt to the persistent CTAs together, so small problems do not pay one launch each.
 */
int64_t qgemm_w4a16_batched_workspace_bytes(int64_t batch, int64_t M, int64_t N, int64_t K);
int qgemm_w4a16_batched(const void* A, const uint8_t* B_packed, const void* scales, int zero, int64_t group, void* C,
                        void* workspace, int64_t workspace_bytes, int64_t batch, int64_t M, int64_t N, int64_t K,
                        int a_dtype, int out_dtype, uint32_t* status, void* stream);

/*
 * W4A16 with the other weight formats of tilelang/quantize: everything as qgemm_w4a16_batched, plus
 *
 * weight_format  QGEMM_W4_SEQUENTIAL: nibble j of a row at byte j/2, bits 4*(j%2) (general_compress,
 *                tilelang/quantize/utils.py:53-69).  QGEMM_W4_INTERLEAVED_F16: every 32-bit word permuted by
 *                interleave_weight(qweight, 4, "float16") (utils.py:73-99): elements 0,2,4,6 in the low
 *                half-word, 1,3,5,7 in the high one, the layout the reference's lop3 decode expects.
 * zeros          nullable fp16 [batch, K/group, N]: one zero point per (group, output feature) instead of the
 *                scalar `zero` (which is then ignored).  Needs scales and N % 16 == 0.
 * zero_mode      how zeros enter (tilelang/quantize/lop3.py:135-175, 232-270, 325-358):
 *                QGEMM_ZERO_ORIGINAL   W = (q - z) * s      (the scalar-zero operators use this form)
 *                QGEMM_ZERO_RESCALE    W = q * s - |z|      (one f16 FMA; needs the zeros tensor)
 *                QGEMM_ZERO_QUANTIZED  W = (q - qz) * s     with integer qz given as fp16 values (unpack
 *                                      packed qzeros on the host first)
 * A zeros tensor of mode QGEMM_ZERO_QUANTIZED (integer zero points 0..15) is taken in flight by the streaming kernel
 * when M <= 64 and the groups are 128 wide, a multiple of 256 or the whole K: no dequantised copy of the weights,
 * (q - qz) exact, and a scratch buffer of qgemm_w4a16_ex_workspace_bytes(..., has_zeros_tensor = 0) suffices.
 * Otherwise a zeros tensor makes the operator dequantise the weights once into the scratch buffer
 * (f16 [batch, N, K]) and multiply with the f16 tensor-core GEMM, whatever the token count; that scratch size comes
 * from qgemm_w4a16_ex_workspace_bytes(..., has_zeros_tensor = 1).  Without a zeros tensor the same kernels as
 * qgemm_w4a16 run.
 */
#define QGEMM_W4_SEQUENTIAL 0
#define QGEMM_W4_INTERLEAVED_F16 1
#define QGEMM_ZERO_ORIGINAL 0
#define QGEMM_ZERO_RESCALE 1
#define QGEMM_ZERO_QUANTIZED 2
int64_t qgemm_w4a16_ex_workspace_bytes(int64_t batch, int64_t M, int64_t N, int64_t K, int has_zeros_tensor);
int qgemm_w4a16_ex(const void* A, const uint8_t* B_packed, const void* scales, const void* zeros, int zero,
                   int zero_mode, int weight_format, int64_t group, void* C, void* workspace, int64_t workspace_bytes,
                   int64_t batch, int64_t M, int64_t N, int64_t K, int a_dtype, int out_dtype, uint32_t* status,
                   void* stream);

/*
 * Gathered W4A16 for weights whose output features are split over several GPUs of one node (one process per
 * GPU): this rank computes its [M, N] block and writes it straight into columns [col0, col0 + N) of n_dst
 * row-major [M, ldc] buffers - its own and every peer's, the peers' mapped into this process with
 * qgemm_ipc_open - with ordinary stores from the kernel's epilogue, so the output crosses NVLink while the
 * rest of the GEMM still runs and no collective has to move or re-arrange it afterwards.  The one-sided
 * counterpart in the reference is the put of src/tl_templates/ascend/common.h:358-408 as used by
 * examples/shmem/shmem_mm_test_put_nbi.py:69-74; there is no gathered dequantize-GEMM in the reference.
 *
 * C_dst is a HOST array of n_dst (1..8) device pointers.  ldc and col0 must be multiples of 8, and from the
 * token count at which the weights are dequantised once (1024) N must be a multiple of 64.  Everything else as
 * qgemm_w4a16 (batch 1, scalar zero point, sequential nibbles); the workspace size is qgemm_w4a16_workspace_bytes.
 * The call returns when the kernels are queued; a destination buffer is complete on its GPU once EVERY rank's
 * call has finished, which the ranks establish among themselves (a stream-ordered barrier, for example a small
 * all-reduce).  No kernel waits for another GPU.
 */
int qgemm_w4a16_gather(const void* A, const uint8_t* B_packed, const void* scales, int zero, int64_t group,
                       void* const* C_dst, int n_dst, int64_t ldc, int64_t col0, void* workspace,
                       int64_t workspace_bytes, int64_t M, int64_t N, int64_t K, int a_dtype, int out_dtype,
                       uint32_t* status, void* stream);

/*
 * Mapping a buffer of another process on the same node into this one, for qgemm_w4a16_gather (no counterpart
 * in the reference, whose SHMEM library owns its symmetric heap).  qgemm_ipc_export fills a
 * QGEMM_IPC_HANDLE_BYTES-byte handle for the device allocation that holds dev_ptr, and the byte offset of
 * dev_ptr inside it; the handle and offset travel to the peer by any host channel; there qgemm_ipc_open maps
 * the allocation and returns its base (add the offset); qgemm_ipc_close unmaps it.  The exporting process
 * must keep the allocation alive while it is mapped elsewhere.
 */
#define QGEMM_IPC_HANDLE_BYTES 64
int qgemm_ipc_export(const void* dev_ptr, void* handle_out, int64_t* offset_out);
int qgemm_ipc_open(const void* handle, void** base_out);
int qgemm_ipc_close(void* base);

/*
 * "Everything I stored into your buffers has landed" between the ranks of the gathered form, without a collective:
 * every rank owns an array of n 32-bit flags (zero-initialised, mapped into all processes like the output buffers);
 * the call stores `epoch` into slot [this rank] of every rank's array (flag_slots[r] = that slot's address in rank
 * r's array, this rank's own included) and then waits until all n slots of its own array (`local_flags`) have reached
 * `epoch` (compared modulo 2^32, so epochs only have to increase by one from call to call).  With `epoch_counter`
 * non-null the epoch is instead that device word (owned by this rank, zero-initialised) incremented by the kernel
 * itself, so that a launch captured in a CUDA graph keeps counting when the graph is replayed; every rank must then
 * execute the same sequence of calls.  One tiny kernel in
 * stream order behind the GEMM launch: the stores of that launch are visible to a peer before the flag is, and the
 * peer's later kernels on its stream run after its own wait.  The wait is bounded by qgemm_set_wait_limit_ms; when it
 * runs out, QGEMM_ST_TIMEOUT_PEER is stored in `status` and the kernel returns.  Replaces the one-element all-reduce
 * that otherwise serves as this barrier (about 12 us at decode sizes).  Ranks must be on different GPUs.
 * No reference counterpart (the reference's analogue is the signal of its one-sided put,
 * src/tl_templates/ascend/common.h:358-408).
 */
int qgemm_peer_signal_wait(void* const* flag_slots, int n, const uint32_t* local_flags, uint32_t epoch,
                           uint32_t* epoch_counter, uint32_t* status, void* stream);

/*
 * W4A16 dequantize-GEMM that needs no memory from the caller beyond inputs and output.  (No counterpart
 * in the reference: there the wrapper allocates every workspace with torch before the call.)
 *
 * Meant for hosts that are not allowed to allocate device memory where the operator runs: an
 * inference-runtime plugin whose execute hook is handed only its tensors and must not call cudaMalloc
 * (the runtime has planned all memory up front, and an allocation there would stall the whole device),
 * or a plain C / FFI caller that owns nothing but its input and output buffers.  Same arguments and
 * results as qgemm_w4a16 without the workspace: the scratch memory is an array inside the library
 * image, QGEMM_W4A16_NOALLOC_SCRATCH_MB megabytes on every GPU that loads the library, held until the
 * process exits.
 *
 * Limits: M <= QGEMM_W4A16_NOALLOC_MAX_M tokens and K <= QGEMM_W4A16_NOALLOC_MAX_K; anything larger is
 * rejected with an error message (use qgemm_w4a16 then).  The function calls no cudaMalloc / cudaFree
 * and no allocating library routine.  The first call on each device looks up the array's device
 * address (one cudaGetSymbolAddress with that device current); make that first call outside any stream
 * capture.  All calls on a device share the one array: it keeps the previous call's contents (every
 * call re-zeroes the counters it needs on the given stream), and two calls that may overlap on the
 * GPU - different streams, or different host threads - race on it and must be serialised by the caller.
 */
#define QGEMM_W4A16_NOALLOC_MAX_M 32
#define QGEMM_W4A16_NOALLOC_MAX_K 16384
#define QGEMM_W4A16_NOALLOC_SCRATCH_MB 6.3
int qgemm_w4a16_noalloc(const void* A, const uint8_t* B_packed, const void* scales, int zero, int64_t group,
                        void* C, int64_t M, int64_t N, int64_t K, int a_dtype, int out_dtype, uint32_t* status,
                        void* stream);

/*
 * int4 -> int8 unpack of a packed weight matrix into a caller-provided [N, K] int8 buffer: the
 * on-device form of torch_unpack_uint4_to_int8 (example_dequant_gemm_fine_grained.py:35-57,
 * signed_nibbles = 0) and of the vector-core unpack stage of w4a8_gemm_cv
 * (examples/dequantize_gemm/example_dequant_gemm_w4a8.py:69-106, signed_nibbles = 1, two's complement).
 */
int qgemm_unpack_int4(const uint8_t* B_packed, int8_t* out, int64_t N, int64_t K, int signed_nibbles,
                      void* stream);

/*
 * W4A8 / int8-mode dequantize-GEMM: C[m,n] = sum_k int32(A[m,k]) * int32(unpack(qB)[n,k]), exact.
 * Replaces kernel(A, qB, workspace, C) of w4a8_gemm_cv (example_dequant_gemm_w4a8.py:25-121; same
 * caller-provided int8 [N, K] workspace) and dequant_gemm_int8_wrapper
 * (example_dequant_gemm_fine_grained.py:226-266).  C is [M, N] int32 (out_dtype must be QGEMM_DT_I32;
 * the reference wrapper casts to other types on the host afterwards, :263).  Requires K % 32 == 0
 * and N % 16 == 0.  Up to 128 tokens the weights are unpacked on their way to the tensor core and the workspace
 * only serves as scratch (its contents after the call are unspecified); above that it receives the int8 copy.
 * Two calls that may overlap on the device must not share a workspace.
 */
int qgemm_w4a8(const int8_t* A, const uint8_t* qB, int8_t* workspace, void* C, int64_t M, int64_t N, int64_t K,
               int signed_nibbles, int out_dtype, uint32_t* status, void* stream);

/*
 * W4A8 with the per-token activation quantiser fused into its pre-pass (decode sizes, M <= 128):
 *   scale_a[m] = max(max_k |X[m,k]|, 1e-4) / 127   (round_scale: rounded up to a power of two)
 *   A[m,k]     = int8(rint(X[m,k] / scale_a[m]))   (never written to memory in the caller's layout)
 *   C[m,n]     = sum_k int32(A[m,k]) * int32(unpack(qB)[n,k])
 * i.e. qgemm_act_quant followed by qgemm_w4a8 in one call, with bit-identical scale_a and C: the reference's
 * act_quant_kernel_int8_optimized (examples/deepseek_v4/act_quant.py:33-92) in front of w4a8_gemm_cv
 * (examples/dequantize_gemm/example_dequant_gemm_w4a8.py:25-121), saving one launch and the int8 round trip.
 * X is [M, K] f16 or bf16, scale_a [M] fp32 (output), workspace the [N, K] int8 scratch of qgemm_w4a8.
 * No reference counterpart as a single operator.
 */
int qgemm_w4a8_act_quant(const void* X, int x_dtype, const uint8_t* qB, int8_t* workspace, int32_t* C, float* scale_a,
                         int round_scale, int64_t M, int64_t N, int64_t K, int signed_nibbles, uint32_t* status,
                         void* stream);

/*
 * Per-token activation quantiser, the step in front of the W8A8 GEMM: it produces that GEMM's A and scale_a.
 * Replaces the compiled `call` of act_quant_kernel_int8_optimized (examples/deepseek_v4/act_quant.py:33-92)
 * and follows its golden act_quant_torch (:112-142) bit for bit:
 *
 *   amax[m] = max(max_n |X[m,n]|, 1e-4)
 *   S[m]    = amax[m] / 127                       (round_scale != 0: 2^ceil(log2(amax[m] / 127)))
 *   Y[m,n]  = int8( round_half_even( clamp(X[m,n] / S[m], -127, 127) ) )
 *
 * X: [M, N] of x_dtype (F16 / BF16), 16-byte aligned.  Y: [M, N] int8.  S: [M] fp32.  Requires N % 8 == 0.
 * A 3-D input [batch, seq, N] is the same call with M = batch * seq.
 */
int qgemm_act_quant(const void* X, int8_t* Y, float* S, int64_t M, int64_t N, int x_dtype, int round_scale,
                    void* stream);

#ifdef __cplusplus
}
#endif
#endif /* QGEMM_H_ */
