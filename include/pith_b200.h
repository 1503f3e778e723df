/*
 * pith_b200 — C ABI of the sm_100a context-parallel attention path.
 *
 * The library replaces the arithmetic behind PithTrain's ring-attention operators
 * (pithtrain/operators/ring_attention/standard.py, pithtrain/operators/ring_attention/mla.py,
 * pithtrain/operators/mla/triton.py). The reference has no foreign-function boundary of its
 * own: its operators call flash-attn and Triton kernels from Python. Each entry point below
 * names the reference call it stands in for.
 *
 * Conventions
 *  - Every buffer is device memory owned by the caller; the library allocates nothing and
 *    keeps no pointer after the call returns. Calls only enqueue work on `stream`.
 *    One exception: pith_attn_bwd_noalloc works in a fixed scratch area that is part of the
 *    library's image on every GPU that loads it (see there).
 *  - Tensors are [B][S][H][D] with the innermost dimension contiguous; strides are given in
 *    ELEMENTS for the b, s and h dimensions. Base pointers and (stride * element size) must
 *    be multiples of 16 bytes. bf16 unless stated.
 *  - LSE / delta tensors are fp32 [B][H][S] with unit stride along S; their b and h strides
 *    are given in elements.
 *  - Return value: 0 = enqueued; negative = rejected on the host (pith_last_error() has the
 *    text). Device-side anomalies (a bounded wait that ran out) are written to *status
 *    (a zero-initialised device uint32, optional) as (code << 24 | detail); see pith_status_string.
 *    Codes: 1 a barrier wait inside a kernel ran out, 2 unexpected TMEM allocation, 3 a wait for a ring neighbour
 *    ran out, 4 a kernel found its shared-memory window misaligned. A launch that finds the word non-zero does no work.
 *  - Re-entrant; no internal threads; no global mutable state besides, per device, one side stream with two
 *    events used by pith_attn_bwd (created on first use) and the device address of the scratch area of
 *    pith_attn_bwd_noalloc (looked up on its first call; it does not survive cudaDeviceReset).
 */
#ifndef PITH_B200_H_
#define PITH_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PITH_B200_ABI_VERSION 2

/* flags for pith_attn_fwd_args.flags */
#define PITH_FWD_O_FP32 1u        /* `o` is fp32 (running accumulator of a ring) instead of bf16 */
#define PITH_FWD_LSE_NATURAL 2u   /* write natural-log LSE (flash-attn convention) instead of log2 */
#define PITH_FWD_SINGLE_CTA 4u    /* use the kernel that runs every MMA inside one CTA */
#define PITH_FWD_CTA_PAIR 8u      /* use the kernel in which pairs of CTAs (thread-block clusters of two) run every MMA
                                     together and each stage half of every K/V block.
                                     Neither flag: the library picks the faster one for the head dimensions (measured:
                                     the pair kernel for Dqk = 192, the single-CTA kernel for Dqk = 128). */

/* flags for pith_attn_bwd_args.flags */
#define PITH_BWD_SERIAL 1u        /* run the dK/dV and dQ passes one after the other on `stream` */
#define PITH_BWD_CONCURRENT 2u    /* run the dQ pass beside the dK/dV pass on a side stream the library keeps per
                                     device, joined into `stream` before the call returns.
                                     Neither flag: the library decides by problem size (side by side for launches of
                                     a few waves, where the partial last wave matters). */

#define PITH_BWD_DQ_STORE_BF16 4u /* `dq_acc` points at a bf16 [B][Sq][Hq][Dqk] OUTPUT (dq_stride in bf16 elements): the dQ
                                     pass stores this block's complete, scaled dQ there instead of adding into an fp32
                                     accumulator. For a backward that consists of this one block (CP = 1): no zero
                                     fill, no final rounding pass. head_dim 128 only. */

/* flags for pith_combine_args.flags */
#define PITH_COMBINE_NATURAL 1u   /* LSEs are natural-log (standard.py) instead of log2 (mla.py) */

/* element types for pith_combine_args.out*_dtype */
#define PITH_DTYPE_BF16 0
#define PITH_DTYPE_F32 1

typedef struct pith_attn_fwd_args {
  const void* q;          /* [B][Sq][Hq][Dqk] bf16 */
  const void* k;          /* [B][Sk][Hkv][Dqk] bf16 */
  const void* v;          /* [B][Sk][Hkv][Dv] bf16 */
  void* o;                /* [B][Sq][Hq][Dv] bf16, or fp32 with PITH_FWD_O_FP32 */
  float* lse;             /* [B][Hq][Sq] */
  const float* prev_o;    /* optional fp32 [B][Sq][Hq][Dv]: partial result to merge in the epilogue */
  const float* prev_lse;  /* optional fp32 [B][Hq][Sq], log2 domain, paired with prev_o */
  uint32_t* status;       /* optional device status word */
  int32_t B, Sq, Sk, Hq, Hkv, Dqk, Dv;
  int32_t causal;         /* 0 = every key visible; 1 = key n visible to query m iff n <= m + causal_offset */
  int32_t causal_offset;
  uint32_t flags;
  float softmax_scale;
  int64_t q_stride[3], k_stride[3], v_stride[3], o_stride[3], prev_o_stride[3]; /* b, s, h (elements) */
  int64_t lse_stride[2], prev_lse_stride[2];                                    /* b, h (elements) */
} pith_attn_fwd_args;

/*
 * Causal / non-causal attention forward for one (Q block, KV block) pair, GQA (Dqk = Dv = 128)
 * or MLA (Dqk = 192, Dv = 128), with log2-domain LSE and an optional fused online-softmax
 * merge with a previous partial (O, LSE).
 * Replaces: flash_attn `_flash_attn_forward` as called at
 *   pithtrain/operators/ring_attention/standard.py:91-93, `flash_attn_func` at
 *   pithtrain/models/qwen3_30b_a3b.py:424, and `_mla_fwd` (pithtrain/operators/mla/triton.py:552-563)
 *   as called at pithtrain/operators/ring_attention/mla.py:67; with prev_o/prev_lse it also covers
 *   the combine at standard.py:94 / mla.py:68.
 */
int pith_attn_fwd(const pith_attn_fwd_args* args, void* stream);

typedef struct pith_bwd_preprocess_args {
  const void* o;    /* [B][S][H][Dv] bf16 */
  const void* dout; /* [B][S][H][Dv] bf16 */
  float* delta;     /* [B][H][S] fp32 = rowsum(o * dout) */
  int32_t B, S, H, Dv;
  int64_t o_stride[3], do_stride[3];
  int64_t delta_stride[2];
} pith_bwd_preprocess_args;

/*
 * delta = rowsum(O * dO).
 * Replaces: `_mla_bwd_preprocess` (pithtrain/operators/mla/triton.py:566-574, kernel :99-122),
 *   called once per backward at pithtrain/operators/ring_attention/mla.py:101; flash-attn computes
 *   the same quantity inside `_flash_attn_backward` (standard.py:134-153).
 */
int pith_attn_bwd_preprocess(const pith_bwd_preprocess_args* args, void* stream);

typedef struct pith_attn_bwd_args {
  const void* q;      /* [B][Sq][Hq][Dqk] bf16 */
  const void* k;      /* [B][Sk][Hkv][Dqk] bf16 */
  const void* v;      /* [B][Sk][Hkv][Dv] bf16 */
  const void* dout;   /* [B][Sq][Hq][Dv] bf16 */
  const float* lse;   /* [B][Hq][Sq] fp32, log2 domain, of the COMPLETE softmax row */
  const float* delta; /* [B][Hq][Sq] fp32 */
  float* dq_acc;      /* [B][Sq][Hq][Dqk] fp32, accumulated into (+=); NULL = skip dQ */
  float* dk_acc;      /* [B][Sk][Hkv][Dqk] fp32, accumulated into (+=); NULL (with dv_acc) = skip dK/dV */
  float* dv_acc;      /* [B][Sk][Hkv][Dv] fp32, accumulated into (+=) */
  uint32_t* status;
  int32_t B, Sq, Sk, Hq, Hkv, Dqk, Dv;
  int32_t causal, causal_offset;
  uint32_t flags;
  float softmax_scale;
  int64_t q_stride[3], k_stride[3], v_stride[3], do_stride[3];
  int64_t dq_stride[3], dk_stride[3], dv_stride[3];
  int64_t lse_stride[2], delta_stride[2];
} pith_attn_bwd_args;

/*
 * dQ, dK, dV contributions of one (Q block, KV block) pair, added into fp32 accumulators so that
 * a ring of steps (and the query heads of one GQA group) round to bf16 once, at the end.
 * Replaces: `_flash_attn_backward` as called at pithtrain/operators/ring_attention/standard.py:134-153
 *   together with the `dq += dq_s` / `local_dk += ...` updates at :154-160,:185-187; and
 *   `_mla_bwd_dk_dv` + `_mla_bwd_dq` (pithtrain/operators/mla/triton.py:577-603) as called at
 *   pithtrain/operators/ring_attention/mla.py:110-115.
 */
int pith_attn_bwd(const pith_attn_bwd_args* args, void* stream);

/*
 * out_bf16[i] = (bf16) acc_f32[i] * scale for a [B][S][H][D] tensor (final rounding of an accumulator).
 * Replaces: the `.to(q.dtype)` at standard.py:104 / mla.py:78 and the implicit bf16 rounding of
 *   flash-attn / Triton gradient outputs.
 */
int pith_cast_f32_to_bf16(const float* acc, void* out, int32_t B, int32_t S, int32_t H, int32_t D,
                          const int64_t acc_stride[3], const int64_t out_stride[3], float scale, void* stream);

typedef struct pith_combine_args {
  const void* out1;  /* [B][S][H][D] */
  const float* lse1; /* [B][H][S] */
  const void* out2;
  const float* lse2;
  float* out;        /* [B][S][H][D] fp32, contiguous */
  float* lse;        /* [B][H][S] fp32, contiguous */
  int32_t out1_dtype, out2_dtype; /* PITH_DTYPE_* */
  int32_t B, S, H, D;
  uint32_t flags;
  int64_t out1_stride[3], out2_stride[3];
  int64_t lse1_stride[2], lse2_stride[2];
} pith_combine_args;

/*
 * Online-softmax merge of two partial attention results.
 * Replaces: `_online_softmax_combine` (pithtrain/operators/ring_attention/standard.py:53-66) and
 *   `_online_softmax_combine_log2` (pithtrain/operators/ring_attention/mla.py:27-40).
 */
int pith_combine(const pith_combine_args* args, void* stream);

#define PITH_MAX_PARTIALS 16

typedef struct pith_partial {
  const void* o;         /* [B][rows][H][D] bf16: attention of query rows [row_begin, row_begin + rows) over one K/V block */
  const float* lse;      /* [B][H][rows] fp32, log2 domain, unit stride along rows */
  int32_t row_begin, rows;
  int64_t o_stride[3];   /* b, s, h strides in elements */
  int64_t lse_stride[2]; /* b, h strides in elements */
} pith_partial;

typedef struct pith_combine_partials_args {
  pith_partial part[PITH_MAX_PARTIALS];
  int32_t n;             /* 1 .. PITH_MAX_PARTIALS */
  int32_t B, S, H, D;
  void* out;             /* [B][S][H][D] bf16, contiguous */
  float* lse;            /* [B][H][S] fp32, contiguous, log2 domain */
} pith_combine_partials_args;

/*
 * Online-softmax merge of up to 16 partial attention results in one pass: every output row is the LSE-weighted mean
 * of the partials that cover it (a row no partial covers, or whose partials all saw no key, gives O = 0, LSE = -inf).
 * Weights and sums are fp32; O is rounded to bf16 once. The forward ring writes one bf16 partial per step and merges
 * them here, instead of carrying an fp32 running result through every step's epilogue.
 * Replaces: the chain of `_online_softmax_combine` / `_online_softmax_combine_log2` calls over the ring steps
 *   (pithtrain/operators/ring_attention/standard.py:94, mla.py:68) and the final `.to(q.dtype)` (standard.py:104).
 */
int pith_combine_partials(const pith_combine_partials_args* args, void* stream);

/* Size of the scratch area built into the library for pith_attn_bwd_noalloc (per GPU, held until exit). */
#define PITH_NOALLOC_SCRATCH_BYTES (32u << 20)

typedef struct pith_attn_bwd_noalloc_args {
  const void* q;     /* [B][Sq][Hq][Dqk] bf16 */
  const void* k;     /* [B][Sk][Hkv][Dqk] bf16 */
  const void* v;     /* [B][Sk][Hkv][Dv] bf16 */
  const void* o;     /* [B][Sq][Hq][Dv] bf16, the forward's output */
  const void* dout;  /* [B][Sq][Hq][Dv] bf16 */
  const float* lse;  /* [B][Hq][Sq] fp32, log2 domain */
  void* dq;          /* [B][Sq][Hq][Dqk] bf16, written */
  void* dk;          /* [B][Sk][Hkv][Dqk] bf16, written */
  void* dv;          /* [B][Sk][Hkv][Dv] bf16, written */
  uint32_t* status;
  int32_t B, Sq, Sk, Hq, Hkv, Dqk, Dv;
  int32_t causal, causal_offset;
  float softmax_scale;
  int64_t q_stride[3], k_stride[3], v_stride[3], o_stride[3], do_stride[3];
  int64_t dq_stride[3], dk_stride[3], dv_stride[3];
  int64_t lse_stride[2];
} pith_attn_bwd_noalloc_args;

/*
 * Complete attention backward (delta, dQ, dK, dV in bf16) that allocates no device memory: delta and the
 * fp32 accumulators live in a PITH_NOALLOC_SCRATCH_BYTES area that is part of the library image.
 * No counterpart in the reference, whose backward helpers allocate their outputs and temporaries through
 * PyTorch. Meant for callers that cannot call cudaMalloc or a framework allocator where the backward runs
 * (frozen memory pools, plugins inside a runtime that owns device allocation, latency-critical loops).
 *  - Problems needing more scratch than the area holds (see pith_attn_bwd_noalloc_scratch_bytes) are
 *    rejected with an error.
 *  - The first call on each device resolves the area's address; make it before any stream capture begins.
 *  - All calls on a GPU share the area: calls whose GPU work overlaps race. Use one stream or order them.
 */
int pith_attn_bwd_noalloc(const pith_attn_bwd_noalloc_args* args, void* stream);
/* Scratch bytes pith_attn_bwd_noalloc needs for a problem (compare with PITH_NOALLOC_SCRATCH_BYTES). */
size_t pith_attn_bwd_noalloc_scratch_bytes(int32_t B, int32_t Sq, int32_t Sk, int32_t Hq, int32_t Hkv, int32_t Dqk,
                                           int32_t Dv);

/*
 * Stream-ordered hand-off flags for moving ring blocks with the copy engines instead of NCCL kernels.
 * Replace: the `req.wait()` on the NCCL requests in `_ring_send_recv_kv`
 *   (pithtrain/operators/ring_attention/standard.py:46-50) and in the dK/dV redistribution (:183-184).
 * Every flag has a sequence counter on each side, in that side's own memory; both start at 0 and advance by one per
 * call, on the device, so the same launches can be replayed from a CUDA graph.
 * pith_flag_signal: in stream order, ++*counter (local memory), publishes all earlier work of `stream` system-wide,
 *   then stores the new *counter into `flag` (which may be mapped memory of a peer GPU).
 * pith_flag_wait: in stream order, ++*counter (local memory), then `stream` waits until the LOCAL `flag` reaches
 *   *counter (wrap-safe). The wait gives up after about `max_seconds` (at most 120), records code 3 in *status and
 *   lets the stream continue; while *status is non-zero every later wait returns at once.
 * pith_enable_peer_access: enables direct access from the current device to `peer_device` (idempotent).
 */
int pith_flag_signal(uint32_t* flag, uint32_t* counter, void* stream);
int pith_flag_wait(const uint32_t* flag, uint32_t* counter, double max_seconds, uint32_t* status, void* stream);
int pith_enable_peer_access(int32_t peer_device);

/*
 * Sharing ring buffers between the processes of one node (CUDA IPC) and copying between them.
 * Replace: `dist.batch_isend_irecv` in `_ring_send_recv_kv` (pithtrain/operators/ring_attention/standard.py:37-45),
 *   which moves the same bytes through NCCL send/recv kernels.
 * pith_ipc_export: writes the 64-byte IPC handle of the device allocation that contains `ptr` into `handle64`
 *   and the byte offset of `ptr` inside that allocation into *offset.
 * pith_ipc_open: maps the allocation behind a handle exported by ANOTHER process into the current device's
 *   address space; *base receives the mapped start of the allocation. One open per handle per process.
 * pith_ipc_close: unmaps what pith_ipc_open returned.
 * pith_peer_copy: enqueues a device-to-device copy of `bytes` on `stream` (copy engine; `src` or `dst` may be
 *   peer-mapped memory).
 */
#define PITH_IPC_HANDLE_BYTES 64
int pith_ipc_export(const void* ptr, void* handle64, uint64_t* offset);
int pith_ipc_open(const void* handle64, void** base);
int pith_ipc_close(void* base);
int pith_peer_copy(void* dst, const void* src, size_t bytes, void* stream);

typedef struct pith_qk_norm_rope_args {
  const void* q;            /* [B][S][Hq][128] bf16 (forward input; the backward recomputes from it) */
  const void* k;            /* [B][S][Hkv][128] bf16 */
  const void* q_weight;     /* [128] RMSNorm weight of the query heads, weight_dtype */
  const void* k_weight;     /* [128] */
  const void* cos;          /* [B][S][128] cs_dtype; a b stride of 0 broadcasts one table over the batch */
  const void* sin;
  void* q_out;              /* forward: rotated queries; backward: dL/dq. bf16 [B][S][Hq][128] */
  void* k_out;              /* forward: rotated keys; backward: dL/dk. bf16 [B][S][Hkv][128] */
  const void* dq_out;       /* backward only: gradient of the rotated queries, bf16 */
  const void* dk_out;       /* backward only: gradient of the rotated keys, bf16 */
  float* dq_weight;         /* backward only: fp32 [128], accumulated into (+=) */
  float* dk_weight;         /* backward only: fp32 [128], accumulated into (+=) */
  int32_t B, S, Hq, Hkv, D; /* D must be 128 */
  int32_t weight_dtype, cs_dtype; /* PITH_DTYPE_* */
  float eps;
  int64_t q_stride[3], k_stride[3], q_out_stride[3], k_out_stride[3], dq_out_stride[3], dk_out_stride[3];
  int64_t cs_stride[2];     /* b, s strides of cos and sin (elements) */
} pith_qk_norm_rope_args;

/*
 * Per-head RMSNorm of Q and K followed by rotary position embedding (rotate-half form), in one pass; and its
 * backward (dL/dq, dL/dk and the two weight gradients) in one pass.
 * Replace: `self.q_norm(...)`, `self.k_norm(...)` (nn.RMSNorm(head_dim), pithtrain/models/qwen3_30b_a3b.py:381-382,
 *   :417-418) and `apply_rotary_pos_emb` (:107-136, called at :421), i.e. two normalisation kernels and eight
 *   elementwise kernels per layer in front of `ring_attention_func` / `flash_attn_func`, and their autograd backward.
 */
int pith_qk_norm_rope_fwd(const pith_qk_norm_rope_args* args, void* stream);
int pith_qk_norm_rope_bwd(const pith_qk_norm_rope_args* args, void* stream);

typedef struct pith_mla_assemble_args {
  /* forward inputs */
  const void* q;       /* [B][S][H][192] bf16: q_nope (128) | q_pe (64, interleaved rotary pairs) */
  const void* kv;      /* [B][S][H][256] bf16: k_nope (128) | v (128) */
  const void* k_pe;    /* [B][S][64] bf16: the one rotary key of a position, shared by all heads */
  const void* cos;     /* [B][S][64] cs_dtype, already gathered by position; a b stride of 0 broadcasts */
  const void* sin;
  /* forward outputs */
  void* query;         /* [B][S][H][192] bf16 */
  void* key;           /* [B][S][H][192] bf16 */
  void* value;         /* [B][S][H][128] bf16 */
  /* backward inputs (gradients of query / key / value; same strides as the forward outputs) */
  const void* dquery;
  const void* dkey;
  const void* dvalue;
  /* backward outputs (same strides as q / kv / k_pe) */
  void* dq;
  void* dkv;
  void* dk_pe;
  int32_t B, S, H;
  int32_t Dnope, Drope, Dv;  /* must be 128, 64, 128 */
  int32_t cs_dtype;          /* PITH_DTYPE_* */
  int64_t q_stride[3], kv_stride[3], query_stride[3], key_stride[3], value_stride[3]; /* b, s, h (elements) */
  int64_t k_pe_stride[2], cs_stride[2];                                                /* b, s (elements) */
} pith_mla_assemble_args;

/*
 * Rotary embedding of the rope parts of Q and K (DeepSeek form) and assembly of the MLA operator's inputs, in one
 * pass; and the backward of it (dk_pe sums over the heads) in one pass.
 * Replace: `apply_rotary_pos_emb` (pithtrain/models/deepseek_v2_lite.py:173-187, called at :446), the four slice
 *   assignments into `new_empty` tensors (:448-454) and `value_states.contiguous()` (:463, :468) in front of
 *   `ring_mla_attention_func` / `MLA`, with their autograd backward.
 */
int pith_mla_assemble_fwd(const pith_mla_assemble_args* args, void* stream);
int pith_mla_assemble_bwd(const pith_mla_assemble_args* args, void* stream);

/* Text of the last host-side rejection on the calling thread. */
const char* pith_last_error(void);
/* Human-readable form of a device status word. Returns a pointer to a thread-local buffer. */
const char* pith_status_string(uint32_t status);
int pith_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* PITH_B200_H_ */
