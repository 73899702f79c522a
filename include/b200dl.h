/* C ABI of libb200dl.so: hand-written sm_100a (B200) kernels for the two dense-contraction
 * hot paths of HugeOrca/sm120-dl, the BF16 GEMM C = A * B^T and the FP16 FlashAttention
 * forward.  Plain pointers and sizes only; every pointer to matrix or tensor data is a
 * DEVICE pointer on the CUDA device that is current when the call is made; `stream` is a
 * cudaStream_t passed as void* (NULL = the legacy default stream).
 *
 * All entry points return 0 on success and a negative B200_E* code on failure; the
 * message of the most recent failure on the calling thread is b200_last_error().
 * Launches are asynchronous on `stream`.  There is no CPU fallback: without an sm_100
 * device the compute entry points fail with B200_ENODEVICE.
 *
 * Each declaration cites the reference interface (path inside HugeOrca/sm120-dl) it
 * stands in for.
 */
#ifndef B200DL_H_
#define B200DL_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_OK 0
#define B200_EINVAL (-1)     /* bad argument: null pointer, unknown config, bad stride      */
#define B200_ESHAPE (-2)     /* shape not supported by the chosen config (divisibility etc.) */
#define B200_ECUDA (-3)      /* a CUDA runtime/driver call failed (sticky error stays set)  */
#define B200_ENODEVICE (-4)  /* current device is not compute capability 10.x               */
#define B200_EDEVICE (-5)    /* a kernel gave up a bounded wait (see b200_device_status)    */

/* ------------------------------------------------------------------ GEMM config registry
 * Replaces the generated table `kGemmConfigs[] / kGemmConfigCount` and the per-config
 * explicit instantiations of gemm_tn<> (gemm/gemm_config_registry.hpp.in:11-37,
 * gemm/gemm_config_registry.cu.in:6-10, gemm/gemm.cu.in:59-66).  The reference runs a config
 * only when M % bm == 0, N % bn == 0 and K % bk == 0 (gemm/test.cpp:449-451) and its
 * registry wrappers keep that rule; the entry points below accept any positive M and K and
 * any positive N that is a multiple of 8 (partial tiles are zero-filled on load and
 * clipped on store by the TMA engine; stores clip at 16-byte granularity, hence N % 8). */
typedef struct b200_gemm_config {
    const char* name;   /* unique, e.g. "bf16_bm256_bn256_bk64_s6_cta2_acc2_bsw8"            */
    int bm;             /* output tile rows per CTA group: 128 * cta_group, or 512 for the "tall"
                           CTA-pair configs, whose CTAs each hold two 128-row accumulators      */
    int bn;             /* output tile columns = N of one tcgen05.mma                        */
    int bk;             /* K extent of one pipeline stage (64 elements = one 128B swizzle)   */
    int stages;         /* depth of the TMA -> MMA shared-memory ring                        */
    int cta_group;      /* 1 = single-CTA MMA, 2 = CTA-pair MMA (cluster of 2 along M)       */
    int acc_bufs;       /* tensor-memory accumulator buffers (2 = epilogue overlaps mainloop) */
    int bs_w;           /* raster: N-tiles per strip, M-major inside a strip                 */
    int smem_bytes;     /* dynamic shared memory per CTA                                     */
    int tmem_cols;      /* tensor-memory columns allocated per CTA                           */
    int split_k;        /* 1, or the cluster size of a split-K config: that many CTAs share one
                           output tile, each accumulating its share of K; the partial tiles are
                           summed through distributed shared memory (no workspace)           */
} b200_gemm_config;

int b200_gemm_num_configs(void);
/* NULL when idx is out of range. */
const b200_gemm_config* b200_gemm_get_config(int idx);
/* Index of the config with exactly this name, or -1. */
int b200_gemm_find_config(const char* name);
/* Index of the config this library would pick for the shape, or -1 for a non-positive
 * shape: the cheapest under a cost model of waves x k-blocks per CTA x tile width over the
 * measured efficiency of that MMA width.  Split-K configs are candidates only when the
 * tiles alone number fewer than 148 and every CTA of the cluster keeps >= 16 k-blocks. */
int b200_gemm_default_config(int M, int N, int K);
/* Stream-K for ragged last waves, off by default.  With mode 1 (process-wide), launches of the
 * persistent configs cut the tiles of a last wave that would leave at least a tenth of the CTA
 * groups idle along K over ALL groups (when every tile has >= 16 k-blocks and there are at
 * least half as many tiles as groups): a group's share is the end of one tail tile (its fp32
 * sums go to a workspace) and the beginning of the next (which it owns: it adds the following
 * groups' sums in a fixed order, so results stay bit-reproducible, and stores the tile).  The
 * workspace comes from a per-device pool (cudaMalloc on first use, ~20 MB; launches that can
 * overlap never share one; at most 8 in flight per device); b200_gemm_bf16_tn_noalloc never
 * cuts.  It is off by default because on B200 it did not pay on the shapes measured: tiles of
 * one wave walk K in lockstep and share their A and B panels through L2, pieces that start
 * at different k-blocks do not, and the fix-up runs at the very end of the kernel where
 * nothing hides it (16384x512x4096: 61 us against 57 us).  No counterpart in the reference
 * (its tile loop hands out whole tiles, gemm/gemm_cute.hpp:121).
 * b200_gemm_uses_stream_k: 1 when a launch of this config and shape would cut its last wave
 * under the current mode on the current device. */
int b200_gemm_set_stream_k(int mode);
int b200_gemm_uses_stream_k(int config, int M, int N, int K);

/* C[M,N] = A[M,K] * B[N,K]^T, bf16 operands, fp32 accumulation, bf16 round-to-nearest-even
 * output, C fully overwritten (alpha = 1, beta = 0).  Row-major with leading dimensions
 * lda, ldb, ldc in ELEMENTS (each a multiple of 8 and at least the row length; the reference
 * has none and means lda = ldb = K, ldc = N).  M, N, K need not be multiples of the tile (N % 8 == 0).  Replaces gemm_tn<T,BM,BN,BK,STAGE,CWG,WARPS_M,WARPS_N,BS_W>
 * (gemm/gemm_cute.hpp:268-356) and the kernel b16_gemm (gemm/gemm_cute.hpp:64-266); the
 * leading dimensions exist so an N-column shard can write its slab of a full-width C. */
int b200_gemm_bf16_tn(int config, int M, int N, int K, const void* A, int64_t lda, const void* B,
                      int64_t ldb, void* C, int64_t ldc, void* stream);

/* The same GEMM for fp16 operands and fp16 output (fp32 accumulation).  The reference's
 * kernel template admits cutlass::half_t (gemm/gemm_cute.hpp:279-280) although its
 * generator only instantiates bf16 (gemm/gemm_configs.py:11-13). */
int b200_gemm_f16_tn(int config, int M, int N, int K, const void* A, int64_t lda, const void* B,
                     int64_t ldb, void* C, int64_t ldc, void* stream);

/* The same GEMM with its result written to n_dst (1..8) destinations: C_list[d] points at the
 * [M,N] window (leading dimension ldc, the same for all) this call owns inside destination
 * d.  Destinations may be on other GPUs of the box (peer-mapped memory): the epilogue stores
 * every finished tile to all of them with TMA over NVLink, so an N-column shard lands in
 * every rank's full-width C while the rest of the GEMM is still running, and no separate
 * all-gather or un-permute copy is needed.  The caller synchronises the ranks afterwards.
 * No counterpart in the reference (it is single-GPU); it replaces the NCCL all-gather the
 * benchmark configuration allows "when the caller needs the full output on one rank". */
int b200_gemm_bf16_tn_scatter(int config, int M, int N, int K, const void* A, int64_t lda,
                              const void* B, int64_t ldb, void* const* C_list, int n_dst, int64_t ldc,
                              void* stream);

/* Same computation, arguments and result as b200_gemm_bf16_tn, for callers that must not
 * allocate device memory: code running after a framework has reserved the whole GPU for its
 * own pool, services with a fixed memory budget that forbid allocation once they are
 * started, and latency-critical loops where an allocator call is not acceptable.  (This
 * entry point has no counterpart in the reference, whose launcher allocates nothing but
 * also keeps no status.)  b200_gemm_bf16_tn allocates a 256-byte status block with
 * cudaMalloc the first time it runs on a device; this variant instead uses a 256-byte
 * array that is part of the library image, so it calls no cudaMalloc, cudaFree or any
 * other allocating routine.  Every GPU that loads the library holds those 256 bytes
 * until the process exits.
 *   - Limit: the array serves at most 256 bytes of scratch per launch; a launch that would
 *     need more is refused with B200_ESHAPE and a message (every current config needs 256).
 *   - The first call on each device resolves the array's device address and reads the
 *     device attributes; make that first call before starting any stream capture.
 *   - All calls share the one array.  Each call clears it on `stream` before its kernel
 *     runs, so calls that overlap on the GPU (different streams) race on it: their results
 *     in C are still correct, but the recorded status is unreliable.  The block written by
 *     this variant is not reported by b200_device_status; read it with
 *     b200_gemm_noalloc_status. */
int b200_gemm_bf16_tn_noalloc(int config, int M, int N, int K, const void* A, int64_t lda,
                              const void* B, int64_t ldb, void* C, int64_t ldc, void* stream);

/* Synchronises the current device and copies out the status word the allocation-free GEMM
 * keeps in its built-in array: 0 when the last b200_gemm_bf16_tn_noalloc launch on this device
 * ran to completion, otherwise the code of the first bounded wait that gave up.  Like that
 * entry point it allocates nothing (one 4-byte copy from the array's address) and has no
 * counterpart in the reference.  The word is cleared by the next noalloc launch, not by
 * this call. */
int b200_gemm_noalloc_status(uint32_t* code);

/* ------------------------------------------------------------- attention config registry
 * Replaces `kFlashFwdConfigs[] / kFlashFwdConfigCount / kFlashFwdDefaultConfigName`
 * (flashattention/v3_mMnNkN/pybind/flash_fwd_config_registry.hpp.in:7-30). */
typedef struct b200_fa_config {
    const char* name;   /* unique, e.g. "hd128_bm64_bn64_tq128x2_tk128_s4_e0_r2"             */
    int head_dim;       /* 64 or 128                                                         */
    int block_m;        /* seq_len must be a multiple of this (query side)                   */
    int block_n;        /* seq_len must be a multiple of this (key side)                     */
    int tile_q;         /* query rows per MMA tile (128)                                     */
    int q_tiles;        /* query tiles processed concurrently by one CTA                     */
    int tile_kv;        /* key/value rows per pipeline stage                                 */
    int stages;         /* depth of the K/V shared-memory ring                               */
    int nwarps;         /* warps per CTA                                                     */
    int smem_bytes;     /* dynamic shared memory per CTA                                     */
    int softmax_layout; /* kernel layout (the trailing _r<n> of the name): 1 = one softmax thread
                           per row that also rescales O, one CTA per 256 query rows; 2 = load,
                           MMA, softmax and correction warpgroups in persistent CTAs, two
                           softmax threads per row; 3 = the same with one softmax thread per row;
                           4 = layout 1 with persistent CTAs (the default)                     */
} b200_fa_config;

int b200_fa_num_configs(void);
const b200_fa_config* b200_fa_get_config(int idx);
int b200_fa_find_config(const char* name);
/* Default config for a head dimension (what fwd() uses), or -1. */
int b200_fa_default_config(int head_dim);

/* O = softmax(Q K^T * softmax_scale [+ causal mask]) V per (batch, head); fp16 in, fp32
 * scores / softmax state / accumulation, fp16 round-to-nearest output.  Tensors are indexed
 * [batch, seq, head, dim] through element strides {stride_b, stride_s, stride_h}; the dim
 * stride is 1; every stride is a multiple of 8 elements.  Causal rule: key j is masked for
 * query i when i < j (top-left aligned, seq_q == seq_k required when causal).
 * Replaces flash_fwd<T,is_causal,H,D,bm,bn,wm,wn,STAGE>
 * (flashattention/v3_mMnNkN/flashatten_v3.hpp:536-573), the kernel flash_atten_v3_fwd
 * (:390-534) and run_flash_fwd_<cfg> (pybind/flash_fwd_config.cu.in:59-91).  The strides
 * exist so a head shard can address its slice of a full [B,S,H,D] tensor. */
int b200_fa_fwd_fp16(int config, const void* q, const void* k, const void* v, void* o, int batch,
                     int seq_q, int seq_k, int heads, int head_dim, const int64_t q_strides[3],
                     const int64_t k_strides[3], const int64_t v_strides[3],
                     const int64_t o_strides[3], float softmax_scale, int causal, void* stream);

/* The same attention with O written to n_dst (1..8) destinations that share o_strides:
 * o_list[d] points at the [batch, seq_q, heads, head_dim] window this call owns inside
 * destination d (for a head shard: the full tensor's base plus the shard's first head).
 * Destinations may be peer-mapped memory of other GPUs; every finished tile is stored to
 * all of them with TMA, so a head shard lands in every rank's full O without an
 * all-gather.  The caller synchronises the ranks afterwards.  No counterpart in the
 * reference (single-GPU). */
int b200_fa_fwd_fp16_scatter(int config, const void* q, const void* k, const void* v, void* const* o_list,
                             int n_dst, int batch, int seq_q, int seq_k, int heads, int head_dim,
                             const int64_t q_strides[3], const int64_t k_strides[3],
                             const int64_t v_strides[3], const int64_t o_strides[3], float softmax_scale,
                             int causal, void* stream);

/* ----------------------------------------------------------------------------- diagnostics */
/* Message of the last failed call on this thread ("" if none). */
const char* b200_last_error(void);
/* Synchronises the current device and reads (then clears) its kernel status word: 0 when
 * every kernel ran to completion, otherwise the code of the first bounded wait that gave
 * up.  Returns B200_OK / B200_ECUDA. */
int b200_device_status(uint32_t* code);
/* Self-test of the bounded waits every kernel of this library uses: launches a one-CTA kernel
 * whose consumer waits for bytes its producer announced and never copied, with a limit of
 * limit_ms (1..1000) milliseconds instead of the kernels' 2 s.  The wait gives up, the
 * kernel returns, and the next b200_device_status() reports the non-zero code 0x80007e57;
 * the device and the library stay usable.  No counterpart in the reference (its waits are
 * unbounded). */
int b200_selftest_wait_expiry(uint32_t limit_ms, void* stream);
/* Library version string. */
const char* b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* B200DL_H_ */
