/*
 * minit_b200 -- C ABI of the B200 (sm_100a) quantized-linear path.
 *
 * Every entry point takes plain device pointers and sizes, launches on the stream it
 * is given (NULL = legacy default stream), never allocates, never synchronises and
 * returns an int status (MT_OK or a negative MT_ERR_*).  Nothing here throws, traps
 * or prints; mt_strerror() turns a status into text.
 *
 * Reference interfaces are cited by their path inside the MiniT project
 * (GetUpEarlier/minit).
 */
#ifndef MINIT_B200_H_
#define MINIT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define MT_OK                 0
#define MT_ERR_NULL          -1  /* a required pointer is NULL */
#define MT_ERR_ALIGN         -2  /* a pointer is not 16-byte aligned */
#define MT_ERR_SHAPE         -3  /* m/n/k/nr_groups violate the layout rules */
#define MT_ERR_DTYPE         -4  /* dtype is not MT_F16 / MT_BF16 */
#define MT_ERR_BITS          -5  /* bits is not 4 or 8 */
#define MT_ERR_WORKSPACE     -6  /* workspace missing or smaller than mt_workspace_bytes() */
#define MT_ERR_CUDA          -7  /* the CUDA runtime reported an error at launch */
#define MT_ERR_UNSUPPORTED   -8  /* valid request that this build has no kernel for */
#define MT_ERR_DEVICE        -9  /* the current device is not compute capability 10.x */
#define MT_ERR_TOO_LARGE    -10  /* request exceeds a fixed built-in capacity */
#define MT_ERR_NCCL         -11  /* the NCCL library reported an error or could not be loaded */
#define MT_ERR_PEER_TIMEOUT -12  /* read back from a workspace error word: a bounded device-side wait expired, the output is not valid */

/* dtype of x / scales / bias / out */
#define MT_F16   0
#define MT_BF16  1

/* flags */
#define MT_FLAG_NONE         0
#define MT_FLAG_FORCE_SMALL  1   /* always use the register-ring streaming kernel (tiles M by 64) */
#define MT_FLAG_FORCE_TC     2   /* always use the tcgen05 kernel */
#define MT_FLAG_FORCE_UMMA  32   /* always use the mid-batch tcgen05 kernel (all warps dequantize; contiguous groups, group size % 64 == 0) */
#define MT_FLAG_FORCE_MID  128   /* always use the integer tensor-core kernel (contiguous groups of a multiple of 128, N % 32 == 0) */
#define MT_FLAG_TC_TMEM_A  256   /* prefill (M > 128, int4): always the 256 x 192 tile with the dequantized weights in tensor memory */
#define MT_FLAG_TC_SMEM_A  512   /* prefill (M > 128, int4): always the 256 x 256 tile with them in shared memory (default: whichever
                                    fills its last wave of tiles better) */
#define MT_FLAG_AR_TWO_SHOT 1024 /* fused all-reduce of 3..32 rows on the integer tensor-core kernel: the two-shot exchange (a column's
                                    partials go to its owner rank, the sum comes back: 2 (w-1)/w of the result's bytes per rank instead of
                                    (w-1) x, two NVLink crossings instead of one).  Same bits as the one-shot form.  Off by default: on four
                                    ranks at 32 rows it measured slower.  Every rank must pass the same flag. */
#define MT_FLAG_AR_ONE_SHOT 2048 /* fused all-reduce: the one-shot exchange even if MT_FLAG_AR_TWO_SHOT is set (the default form) */
#define MT_FLAG_FORCE_VEC   16   /* always use the CUDA-core decode GEMV (M <= 2, contiguous groups, N % 128 == 0) */
#define MT_FLAG_SPLITS(s)   (((s) & 0xff) << 16)   /* tuning: force the split-K factor of the decode GEMV */
#define MT_FLAG_PDL          4   /* launch with programmatic stream serialization: the kernel starts
                                    fetching weights before the previous kernel in the stream ends and
                                    waits for it only before touching x / out / workspace */
#define MT_FLAG_AR_SHORT_WAIT 64 /* fused all-reduce: give up on a peer after ~4 thousand polls (a fraction of a
                                    millisecond) instead of ~4 million; for tests of the time-out path */

/* Library version: major*10000 + minor*100 + patch. */
int mt_version(void);

/* Text for a status code (static storage). */
const char* mt_strerror(int status);

/*
 * Bytes of workspace mt_qgemm / mt_w8_perchannel_gemm need for a problem size.  The
 * caller owns the buffer, must zero it once after allocation (the kernels leave it
 * zeroed) and must not share it between streams that run concurrently.
 */
size_t mt_workspace_bytes(int m, int n, int k, int bits);

/*
 * W[k,n] = (T(q[k,n]) - (T(z[g(k),n]) + 1)) * s[g(k),n], written as [K,N] row-major in T.
 * Replaces the reference's unpack() (examples/qwen1_5_int8.py:40-50) followed by
 * Dequantize / dispatch_dequantize (minit/quantize/operator.py:5-7,
 * minit/quantize/dispatch.py:14-20), bit-exactly.
 *   qweight  uint32 [K/(32/bits), N]  element k at bits ((k % pack)*bits) of word k/pack
 *   g_idx    int32  [K] or NULL (NULL: g(k) = k / (K/nr_groups))
 *   qzeros   uint32 [nr_groups, N/(32/bits)] or NULL (NULL: stored zero = 2^(bits-1) - 1)
 *   scales   T      [nr_groups, N]
 * Rules: n % 8 == 0, k % 32 == 0, all pointers 16-byte aligned.
 */
int mt_dequant(void* stream, const uint32_t* qweight, const int32_t* g_idx, const uint32_t* qzeros,
               const void* scales, void* w_out, int n, int k, int nr_groups, int bits, int dtype);

/*
 * Same formula on UNPACKED operands, the form the reference's QuantizedTensor holds
 * (minit/quantize/tensor.py:9-30: data [K,N] uint8, group [K] int32, zero [G,N] uint8,
 * scale [G,N] T) and dequantize(x, group, zero, scale, axis=0) consumes
 * (minit/quantize/functional.py:6-8).  g_idx NULL: g(k) = k / (K/nr_groups).  n % 4 == 0.
 */
int mt_dequant_unpacked(void* stream, const uint8_t* q, const int32_t* g_idx, const uint8_t* z,
                        const void* scales, void* w_out, int n, int k, int nr_groups, int dtype);

/*
 * int32-packed -> one element per byte: the reference's unpack(x, axis)
 * (examples/qwen1_5_int8.py:40-50), extended to 4-bit with the accessor formula of
 * ColPackedMatrix / RowPackedMatrix (examples/qwen1_5_int8.py:97-138).  rows/cols are the
 * UNPACKED sizes; axis 0: packed is [rows/pack, cols]; axis 1: packed is [rows, cols/pack].
 */
int mt_unpack(void* stream, const uint32_t* packed, uint8_t* out, int rows, int cols, int bits, int axis);

/*
 * out[M,N] = x[M,K] @ W[K,N] (+ bias[N]), W as defined by mt_dequant, fp32 accumulation,
 * result rounded once to T.  Replaces the reference's fused kernel launcher
 *   extern "C" void qmm_<name>(cudaStream_t, T* x, unsigned* qweight, int* g_idx, unsigned* zeros,
 *                              T* scales, TOut* outputs, int m, int n, int k, int nr_groups)
 * (examples/qwen1_5_int8.py:202-216, kernel :156-200) with the same argument order, extended
 * by bias, bits, dtype, workspace and flags.  Differences a caller must know: out is
 * OVERWRITTEN (the reference accumulates into a pre-zeroed buffer), and the int return
 * replaces exceptions / traps.
 * Rules: as mt_dequant; without g_idx the group size K/nr_groups must be a multiple of 32;
 * workspace >= mt_workspace_bytes(m, n, k, bits).
 */
int mt_qgemm(void* stream, const void* x, const uint32_t* qweight, const int32_t* g_idx,
             const uint32_t* qzeros, const void* scales, const void* bias, void* out,
             int m, int n, int k, int nr_groups, int bits, int dtype,
             void* workspace, size_t workspace_bytes, int flags);

/*
 * Row-parallel linear with the all-reduce fused into the GEMM epilogue: out[M,N] on EVERY rank =
 * sum over ranks of (x_r[M,K_r] @ W_r[K_r,N]) (+ bias, pass it on one rank only).  Replaces the pair
 * "local matmul, then Partial -> all_reduce" of the reference (minit/collective/dispatch.py:33-37,
 * minit/collective/tensor.py:72-73, ncclAllReduce at minit/nccl/kernel.py:51-53) with one kernel:
 * the thread that finishes four fp32 partials of a row pushes them, each paired with the call's
 * sequence number, into its mailbox in every peer's symmetric buffer with plain peer stores, then
 * polls (bounded; on expiry the workspace error word is set to 4) the peers' mailboxes in its own
 * memory and sums over all ranks in rank order.  One NVLink crossing per value, no fence, no
 * NCCL call, no multicast; results are bit-identical on all ranks.
 *   peer_buffers  DEVICE array [world] of pointers: entry r is rank r's symmetric buffer as mapped
 *                 into this process (entry `rank` is the local one).  Every buffer has buffer_bytes
 *                 >= mt_allreduce_buffer_bytes(m_max, n_max, world) and must be zero before first use.
 *   All ranks must issue the same sequence of calls on the same buffers; m <= 64 per call.
 * world == 1 degenerates to mt_qgemm on the streaming kernel.
 */
int mt_qgemm_allreduce(void* stream, const void* x, const uint32_t* qweight, const int32_t* g_idx,
                       const uint32_t* qzeros, const void* scales, const void* bias, void* out,
                       int m, int n, int k, int nr_groups, int bits, int dtype,
                       void* workspace, size_t workspace_bytes, int flags,
                       void* const* peer_buffers, int rank, int world, size_t buffer_bytes);

/*
 * Several decode linears (M <= 2) of a layer in ONE launch, in list order.  Replaces a run of fused-kernel launches
 * of the reference (examples/qwen1_5_int8.py:244-267 calls its launcher once per linear; a decoder layer issues
 * q/k/v, o, gate/up, down back to back) and, for row-parallel entries, the all_reduce after each of them
 * (minit/nccl/kernel.py:51-53).  An entry may read what an EARLIER entry of the same call wrote (x or residual
 * = an earlier out): before a warp reads its activations it waits -- bounded; on expiry the workspace error word
 * is set to 6 -- until every column block of the earlier entries is stored.  The weights do not wait: the grid is
 * resident as a whole and the first rows of the next entry are requested before the previous entry's partial sums
 * are combined, so the weight stream does not stop between linears.
 *   Every entry must be a request the decode GEMV accepts: no g_idx, N % 128 == 0, group size % 32 == 0 (all
 *   entries of a call with the same group size class: all % 64 == 0, or none).  m, bits, dtype, workspace and the
 *   peers are shared.  epilogue: MT_EPILOGUE_NONE or MT_EPILOGUE_SWIGLU (out is [M, N/2]).  allreduce != 0: the
 *   entry's finished sums are exchanged over peer_buffers as in mt_qgemm_allreduce (residual added after the sum).
 *   count <= MT_CHAIN_MAX.  The launch is cooperative: it fails with MT_ERR_CUDA rather than wait for CTAs that
 *   cannot be resident.  Returns MT_ERR_UNSUPPORTED when the list does not fit; the caller then issues the
 *   linears one by one.
 */
#define MT_CHAIN_MAX 16
typedef struct mt_chain_linear {
    const void* x;             /* [M,K] T */
    const uint32_t* qweight;   /* [K/pack, N] */
    const uint32_t* qzeros;    /* [G, N/pack] or null */
    const void* scales;        /* [G, N] T */
    const void* bias;          /* [N] T or null */
    const void* residual;      /* [M,N] T or null */
    void* out;                 /* [M,N] T ([M,N/2] with MT_EPILOGUE_SWIGLU) */
    int n, k, nr_groups;
    int epilogue;
    int allreduce;
} mt_chain_linear;
int mt_qgemm_chain(void* stream, const mt_chain_linear* linears, int count, int m, int bits, int dtype,
                   void* workspace, size_t workspace_bytes, int flags,
                   void* const* peer_buffers, int rank, int world, size_t buffer_bytes);
size_t mt_allreduce_buffer_bytes(int m_max, int n_max, int world);

/*
 * Epilogues of a decoder layer fused into the linear (the reference runs each as separate elementwise
 * kernels on the linear's rounded output):
 *
 * mt_qgemm_residual: out[M,N] = residual[M,N] + (x @ W (+ bias)), the `x + attention_output` /
 *   `x + feed_forward_output` of a decoder block (examples/llama3_70b.py:160).  With world > 1 it is
 *   mt_qgemm_allreduce (same buffers and rules, m <= 64) with the residual, replicated on every rank,
 *   added to the reduced sum; with world <= 1 peer_buffers is ignored and any m is accepted.  At M <= 2
 *   the decode GEMV adds the residual in fp32 before its one rounding; other batch sizes run the GEMM,
 *   then one elementwise launch (two roundings, as in the reference).  residual must not overlap out
 *   unless M <= 2; residual NULL = mt_qgemm / mt_qgemm_allreduce.
 *
 * mt_interleave_gate_up (load time): the gate and up projections of a gated feed-forward
 *   (examples/llama3_70b.py:118-130, examples/qwen1_5_int8.py:371-383), each [K, n_half] in the GPTQ layout
 *   with the same K, groups and bits, become ONE linear of N = 2 n_half columns: output column c holds
 *   gate column 4 (c / 8) + c % 8 if c % 8 < 4, else up column 4 (c / 8) + c % 8 - 4.  qzeros and bias
 *   are optional (all three pointers of a kind NULL or none); n_half % 8 == 0.  Not in place.
 *
 * mt_qgemm_swiglu: out[M, N/2] = silu(G) * U where [G | U] = x @ W (+ bias) on that interleaved
 *   layout: out[m, j] = silu(y[m, 8 (j / 4) + j % 4]) * y[m, 8 (j / 4) + 4 + j % 4], computed in fp32
 *   and rounded once (the reference rounds the linear outputs, sigmoid, silu and the product separately:
 *   Sigmoid rule at minit/cuda/dispatch.py:143).  At M <= 2 it runs in the epilogue of the decode GEMV;
 *   otherwise the GEMM writes y into scratch ([M,N], required then) and mt_swiglu follows.  N % 16 == 0,
 *   no act-order.
 *
 * mt_swiglu: the activation alone, gate_up[M,N] interleaved -> out[M,N/2].
 */
#define MT_EPILOGUE_NONE    0
#define MT_EPILOGUE_SWIGLU  1
int mt_qgemm_residual(void* stream, const void* x, const uint32_t* qweight, const int32_t* g_idx,
                      const uint32_t* qzeros, const void* scales, const void* bias, const void* residual, void* out,
                      int m, int n, int k, int nr_groups, int bits, int dtype,
                      void* workspace, size_t workspace_bytes, int flags,
                      void* const* peer_buffers, int rank, int world, size_t buffer_bytes);
int mt_interleave_gate_up(void* stream, const uint32_t* gate_qweight, const uint32_t* up_qweight,
                          const uint32_t* gate_qzeros, const uint32_t* up_qzeros, const void* gate_scales, const void* up_scales,
                          const void* gate_bias, const void* up_bias,
                          uint32_t* qweight_out, uint32_t* qzeros_out, void* scales_out, void* bias_out,
                          int n_half, int k, int nr_groups, int bits);
int mt_qgemm_swiglu(void* stream, const void* x, const uint32_t* qweight, const uint32_t* qzeros, const void* scales,
                    const void* bias, void* out, void* scratch, int m, int n, int k, int nr_groups, int bits, int dtype,
                    void* workspace, size_t workspace_bytes, int flags);
int mt_swiglu(void* stream, const void* gate_up, void* out, int m, int n, int dtype);

/*
 * The steps either side of the linears in a decoder layer, for decode-sized batches of ONE sequence
 * (m new tokens at positions offset .. offset + m - 1, as in the reference's examples):
 *
 * mt_rms_norm: out[r, :] = T(float(x[r, :]) / sqrt(mean(x[r, :]^2) + eps) * float(weight)), the kernel of
 *   minit/cuda/kernel/cuda/rms_norm.py:55-91 for the last axis.  h % 8 == 0.
 *
 * mt_rope_append: rotary embedding and cache append for one fused qkv row per token,
 *   qkv[m, (hq + 2 hkv) * d] = [q heads | k heads | v heads].  Pairs (x[2i], x[2i+1]) of every q and k head are
 *   rotated by (cos, sin)[position, i] in fp32 (minit/cuda/kernel/cuda/rope.py:58-73; tables fp32
 *   [table_rows, d/2]); q goes to q_out[m, hq, d], k and v to k_cache / v_cache[capacity, hkv, d] at row
 *   offset + token.  This replaces rope + F.tie of examples/llama3_70b.py:97-102: the cache is preallocated
 *   and holds every kv head once (the reference stores it nr_groups times, :85-94).  Any even d.
 *   offset_dev (device int32, may be NULL) overrides `offset` so that a captured graph can be replayed as
 *   the sequence grows; rows beyond capacity are not written.
 *
 * mt_attention_decode: out[m, hq * d] = softmax(q k^T * scale + causal mask) v against the cache rows
 *   0 .. offset + token (examples/llama3_70b.py:103-115), query head n reading kv head n / (hq / hkv).
 *   One kernel, fp32 throughout, one rounding (the reference rounds scores, scaled scores, probabilities
 *   and output separately).  max_len bounds offset + m (the grid is sized for it; pass the cache capacity
 *   with offset_dev).  d == 128, hq / hkv <= 8.  workspace >= mt_attention_workspace_bytes(m, hkv, max_len),
 *   zeroed once by the caller (the kernel leaves it zeroed).
 */
int mt_rms_norm(void* stream, const void* x, const void* weight, void* out, int rows, int h, float eps, int dtype);
int mt_rope_append(void* stream, const void* qkv, const float* cos_table, const float* sin_table, void* q_out, void* k_cache, void* v_cache,
                   int m, int hq, int hkv, int d, int offset, const int32_t* offset_dev, int capacity, int table_rows, int dtype);
/*
 * mt_qgemm_rope_append: the fused q/k/v linear of a decode step with mt_rope_append as its epilogue:
 * qkv = x @ W (+ bias) with W[K, (hq + 2 hkv) * d], rotated and scattered to q_out / k_cache / v_cache without ever
 * being stored as a row.  At M <= 2 (decode GEMV) the rotation runs on the fp32 sums, one rounding; otherwise the
 * GEMM writes the row into scratch ([M, (hq + 2 hkv) d], required then) and mt_rope_append follows.  No act-order.
 */
int mt_qgemm_rope_append(void* stream, const void* x, const uint32_t* qweight, const uint32_t* qzeros, const void* scales, const void* bias,
                         const float* cos_table, const float* sin_table, void* q_out, void* k_cache, void* v_cache, void* scratch,
                         int m, int hq, int hkv, int d, int k, int nr_groups, int bits, int dtype,
                         int offset, const int32_t* offset_dev, int capacity, int table_rows,
                         void* workspace, size_t workspace_bytes, int flags);
/*
 * mt_attention: the same attention for prefill-sized and multi-sequence batches and for any head size that is a multiple
 *   of 32 up to 256 (examples/llama3_70b.py:103-115: all (query, key) scores, the causal mask shifted by the cached
 *   positions, softmax over the keys, weighted sum of the values; minit/cuda/kernel/cuda/softmax.py:55-114).
 *   q[batch, m, hq, d] (rotated), k_cache / v_cache[batch, capacity, hkv, d] holding positions 0 .. offset_b + m - 1 of every
 *   sequence, out[batch, m, hq * d]; query i of sequence b sits at position offset_b + i and sees keys 0 .. offset_b + i.
 *   offsets_dev (device int32 [batch], may be NULL) gives every sequence its own offset_b, else `offset` holds for all.
 *   fp32 throughout, one rounding.  mt_rope_append (any even d) fills the cache of one sequence at a time.
 */
int mt_attention(void* stream, const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* offsets_dev,
                 int batch, int m, int hq, int hkv, int d, int offset, int capacity, float scale, int dtype);
size_t mt_attention_workspace_bytes(int m, int hkv, int max_len);
int mt_attention_decode(void* stream, const void* q, const void* k_cache, const void* v_cache, void* out, int m, int hq, int hkv, int d,
                        int offset, const int32_t* offset_dev, int max_len, float scale, void* workspace, size_t workspace_bytes, int dtype);

/*
 * Which schedule mt_qgemm would run a decode call (M <= 2, no g_idx) with: > 0 = split-K factor of the
 * CUDA-core GEMV, 0 = its stream-K schedule, MT_ERR_UNSUPPORTED = the request goes to another kernel.
 * Inspection only (no launch); no counterpart in the reference, whose launcher has one fixed grid
 * (examples/qwen1_5_int8.py:202-216).
 */
int mt_decode_plan(int m, int n, int k, int nr_groups, int bits, size_t workspace_bytes, int flags);

/*
 * mt_qgemm for callers that cannot allocate.  No counterpart in the reference (its launcher
 * needs no scratch because it accumulates with atomics into a pre-zeroed output).
 *
 * Same computation and argument meaning as mt_qgemm, always on the streaming kernel, but the
 * split-K scratch is a fixed MT_STATIC_SCRATCH_BYTES array inside the library instead of a
 * caller-supplied workspace; this call and everything under it allocates nothing.  It is meant
 * for hosts that have given all device memory to their own pool (a later cudaMalloc by a
 * library would fail) or that cannot tolerate the synchronisation an allocation implies inside
 * a decode loop.  Every GPU that loads the library holds the array until the process exits.
 *   - Limit: refused with MT_ERR_TOO_LARGE when mt_workspace_bytes(m, n, k, bits) exceeds
 *     MT_STATIC_SCRATCH_BYTES (e.g. int4 K = N = 8192 fits, K = 8192 x N = 57344 does not).
 *   - The first call on a device looks up the array's device address.  With CUDA's default lazy
 *     module loading that look-up is also the moment the driver loads the module that holds the
 *     array and reserves its MT_STATIC_SCRATCH_BYTES on that device (under
 *     CUDA_MODULE_LOADING=EAGER this happens when the library is loaded instead).  So make one
 *     call per device at start-up: BEFORE the host claims the remaining device memory for its
 *     own pool (afterwards the reservation would fail and the call returns MT_ERR_CUDA) and
 *     before starting any stream capture on that device.  Later calls reserve nothing.
 *   - All calls on a device share the one array (it keeps the previous call's contents; the
 *     part that must start at zero is cleared on `stream` by each call).  Two calls that can
 *     overlap on the GPU -- different streams, no dependency -- race on it: serialise them.
 *   - MT_FLAG_PDL and MT_FLAG_FORCE_TC are ignored.
 */
#define MT_STATIC_SCRATCH_BYTES (8u << 20)
int mt_qgemm_static(void* stream, const void* x, const uint32_t* qweight, const int32_t* g_idx,
                    const uint32_t* qzeros, const void* scales, const void* bias, void* out,
                    int m, int n, int k, int nr_groups, int bits, int dtype, int flags);

/*
 * out[M,N] = (x[M,K] @ float(w[K,N])) * scales[N] (+ bias[N]): int8 weight-only, one scale
 * per output channel.  This is the G = 1, g_idx = 0, stored-zero = 127, q = w + 128 special
 * case of the formula above (minit/quantize/dispatch.py:14-20) with w kept as plain int8
 * [K,N] row-major instead of packed words.
 * Rules: n % 16 == 0, k % 16 == 0, pointers 16-byte aligned.
 */
int mt_w8_perchannel_gemm(void* stream, const void* x, const int8_t* w, const void* scales,
                          const void* bias, void* out, int m, int n, int k, int dtype,
                          void* workspace, size_t workspace_bytes, int flags);

/*
 * mt_w8_pack: plain int8 weights w[K,N] -> the 8-bit GPTQ word layout qweight[K/4, N] (byte i of word
 * (kw, n) = w[4 kw + i][n] + 128).  A per-channel int8 linear is then mt_qgemm(bits = 8, nr_groups = 1,
 * qzeros = NULL, scales [1,N]) and runs on the same kernels as a GPTQ linear (CUDA-core GEMV at M <= 2,
 * tcgen05 at M > 64); mt_w8_perchannel_gemm on the plain layout remains for callers that cannot repack.
 * Load-time; n % 4 == 0, k % 4 == 0.
 */
int mt_w8_pack(void* stream, const int8_t* w, uint32_t* qweight, int n, int k);

/*
 * Act-order (desc_act) checkpoints: g_idx[k] is the group of row k, in arbitrary order
 * (examples/qwen1_5_int8.py:97-138 looks scales and zeros up through it for every element).  Sorted
 * once by group, the weights have the contiguous-group layout of all fast kernels, and the
 * activations are read through the same permutation: x[:, perm] @ W[perm, :] == x @ W.
 *   mt_act_order_perm    perm[K] = stable argsort of g_idx; *status (device int, may be NULL) = 0 ok,
 *                        1 a group does not hold exactly K / nr_groups rows, 2 a g_idx value out of range.
 *   mt_repack_rows       qweight_out row r = qweight row perm[r] (inside the packed words; not in place).
 *   mt_gather_columns    x_out[m, j] = x[m, perm[j]].
 *   mt_qgemm_ordered     out = x[:, x_perm] @ dequant(qweight sorted, contiguous groups) (+ bias).  At
 *                        M <= 2 the GEMV gathers while it stages x; otherwise x is gathered into
 *                        x_scratch ([M,K], required then) by one extra launch.  x_perm NULL = mt_qgemm.
 * Load-time functions may be called once per layer; none allocates or synchronises.
 */
int mt_act_order_perm(void* stream, const int32_t* g_idx, int32_t* perm, int* status, int k, int nr_groups);
int mt_repack_rows(void* stream, const uint32_t* qweight, const int32_t* perm, uint32_t* qweight_out, int n, int k, int bits);
int mt_gather_columns(void* stream, const void* x, const int32_t* perm, void* x_out, int m, int k, int dtype);
int mt_qgemm_ordered(void* stream, const void* x, const int32_t* x_perm, void* x_scratch, const uint32_t* qweight,
                     const uint32_t* qzeros, const void* scales, const void* bias, void* out,
                     int m, int n, int k, int nr_groups, int bits, int dtype,
                     void* workspace, size_t workspace_bytes, int flags);

/*
 * NCCL plumbing with the reference's entry-point names (minit/nccl/library.py:41-58,
 * minit/nccl/kernel.py:47-57), returning a status instead of throwing.  libnccl is
 * opened with dlopen() on first use: mt_nccl_load(path) selects the file (NULL:
 * "libnccl.so.2").  dtype: MT_F16 / MT_BF16, or 2 = float32, 3 = int32.
 */
int    mt_nccl_load(const char* path);
size_t nccl_unique_id_size(void);
int    nccl_create_unique_id(char* bytes);
int    nccl_init_rank(int nr_ranks, int rank, const char* bytes, int device, void** comm_out);
int    nccl_destroy(void* comm);
int    nccl_all_gather(void* stream, void* comm, const void* sendbuff, void* recvbuff, size_t count, int dtype);
int    nccl_all_reduce(void* stream, void* comm, const void* sendbuff, void* recvbuff, size_t count, int dtype);
int    nccl_broadcast(void* stream, void* comm, const void* sendbuff, void* recvbuff, size_t count, int dtype, int root);

#ifdef __cplusplus
}
#endif
#endif /* MINIT_B200_H_ */
