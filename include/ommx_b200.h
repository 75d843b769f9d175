/*
 * ommx_b200.h - C ABI of libommx_b200.so: OMMX paged decode attention over a quantized KV
 * cache, hand-written for NVIDIA B200 (sm_100a).
 *
 * The library replaces three pieces of Youngmin17/open_ommx_serve behind their own Python
 * entry points; each function below names the reference interface it stands in for (paths are
 * relative to the reference checkout).  Every pointer is a plain device pointer unless the
 * comment says "host".  Every function returns 0 on success or a negative OMMX_E_* code when
 * an argument is rejected on the host before anything is launched; ommx_b200_last_error()
 * then gives the reason as text.  Kernels never trap: out-of-range page or group-slot ids, a
 * non-finite value handed to the packer or a wait that ran out are reported through the
 * optional `status` word (device int32, OR-ed OMMX_ST_* bits) and the access is skipped.
 * `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 */
#ifndef OMMX_B200_H_
#define OMMX_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OMMX_B200_ABI_VERSION 4

/* host-side argument errors (return values) */
#define OMMX_E_ARG          (-1)   /* null pointer, bad size, misaligned plane */
#define OMMX_E_UNSUPPORTED  (-2)   /* a geometry/recipe this build does not implement */
#define OMMX_E_CUDA         (-3)   /* a CUDA runtime call failed (launch, attribute) */

/* device status bits (OR-ed into *status) */
#define OMMX_ST_BAD_PAGE     1     /* page id outside [0, num_pages) - access skipped */
#define OMMX_ST_BAD_GROUP    2     /* group slot outside [0, num_group_slots) - access skipped */
#define OMMX_ST_NONFINITE    4     /* packer saw NaN/Inf in K or V */
#define OMMX_ST_TIMEOUT      8     /* a bounded wait inside a kernel ran out */
#define OMMX_ST_BAD_LENGTH  16     /* b_seq_len needs more groups per split than a CTA can index */
#define OMMX_ST_SCALE_RANGE 32     /* a K or V scale exponent above 11 was clamped in decode (scale step > 2048) */

/* element types of q / o / k,v inputs */
#define OMMX_DT_F32   0
#define OMMX_DT_BF16  1
#define OMMX_DT_F16   2

/* outlier-index plane encoding (ommx_kv_planes.outlier_index) */
#define OMMX_OIDX_BITMASK 0
#define OMMX_OIDX_RELIDX7 1

/* how k_scale / v_scale are stored */
#define OMMX_SCALE_INT8_EXP 0      /* int8 power-of-two exponent (the serving default) */
#define OMMX_SCALE_BF16     1
#define OMMX_SCALE_F32      2

/*
 * The packed KV planes (reference ABI: ommx_gpu_serve/attention/paged_decode.py:2856-2887,
 * produced by ommx_gpu_serve/attention/pack.py:628-655).  All planes are contiguous.
 *   k_base / v_main   u8  [num_pages, page_size, n_kv_heads, head_dim/4]   2-bit codes
 *   v_scale           i8|bf16|f32 [num_pages, page_size, n_kv_heads, head_dim/32]
 *   v_zp              bf16|f32    [num_pages, page_size, n_kv_heads, head_dim/32]
 *   k_scale           i8|bf16|f32 [num_group_slots, n_kv_heads, head_dim]
 *   k_zp, k_mapscale, k_mapcenter  bf16|f32 [num_group_slots, n_kv_heads, head_dim]
 *   k_obmp            u8  [num_group_slots, n_kv_heads, head_dim, 4]   bit p = token p (LSB first)
 *   k_oval            u8  [num_group_slots, n_kv_heads, head_dim, ceil(k/2)]  FP4 nibbles,
 *                                                       nibble s = s-th outlier in token order
 * A "group" is 32 consecutive tokens; a K vector is (head, channel, group), a V vector is
 * (token, head, 32 consecutive channels).
 */
typedef struct ommx_kv_planes {
    int32_t n_kv_heads;
    int32_t head_dim;
    int32_t page_size;            /* tokens per page: 8, 16 or 32 */
    int32_t num_pages;
    int32_t num_group_slots;
    int32_t outliers_per_vector;  /* k: FP4 outliers per 32-token K vector (pack and decode: 0..16; the decode-step store: 0, 2, 4, 6, 8) */
    int32_t kv_outlier_map;       /* 1: outliers use k_mapscale/k_mapcenter, 0: share scale/zp */
    int32_t scale_kind;           /* OMMX_SCALE_* (zp and map planes are f32 iff OMMX_SCALE_F32) */
    void *k_base, *k_scale, *k_zp, *k_obmp, *k_oval, *k_mapscale, *k_mapcenter;
    void *v_main, *v_scale, *v_zp;
    int32_t outlier_index;        /* what k_obmp holds per (group, head, channel) frame: OMMX_OIDX_BITMASK = 4 bytes, bit p
                                     set iff token p is an outlier (attention/codec.py:330-372); OMMX_OIDX_RELIDX7 = the
                                     reference's relidx7 stream, ceil(7k/8) bytes of 7-bit token positions, ascending,
                                     LSB first (attention/codec.py:91-130, its k_oidx plane).  Decode reads both; the
                                     store kernels write the bitmask (ommx_b200_outlier_index_convert makes the other). */
} ommx_kv_planes;

/*
 * KV quantize + pack ("store").  Replaces ommx_pack_kv_canonical_block
 * (ommx_gpu_serve/attention/pack.py:293-655) and the per-slot plane copies its callers do
 * afterwards (attention/kv_store.py:594-610, attention/kv_pool.py:619-635): the block of
 * num_tokens = 32*n rows is quantized and written straight into the destination pages and
 * group slots.  Output is bit-identical to the reference packer run on CPU.
 */
typedef struct ommx_pack_args {
    const void *k, *v;            /* [num_tokens, n_kv_heads, head_dim], last dim contiguous */
    int32_t in_dtype;             /* OMMX_DT_* */
    int32_t num_tokens;           /* multiple of 32 and of page_size */
    int64_t stride_token, stride_head;   /* in elements, shared by k and v */
    const int32_t *dst_pages;     /* [num_tokens/page_size] destination page ids, NULL = 0,1,2.. */
    const int32_t *dst_groups;    /* [num_tokens/32] destination group slots,  NULL = 0,1,2.. */
    int32_t outlier_select;       /* 1 = signed (top ceil(k/2) + bottom floor(k/2)), 0 = abs */
    int32_t use_pow2;             /* 1 = snap scales to powers of two */
    ommx_kv_planes planes;        /* destination */
    int32_t *status;              /* optional */
} ommx_pack_args;

int ommx_b200_pack_kv(const ommx_pack_args *args, void *stream);

/*
 * Re-encode an outlier-index plane of `frames` (group, head, channel) frames with k outliers each between the
 * flat bitmask (4 bytes per frame) and relidx7 (ceil(7k/8) bytes per frame): to_relidx7 = 1 bitmask -> relidx7,
 * 0 the other way.  Replaces _pack_relidx7_frames / _unpack_relidx7_streams (attention/pack.py:128-176) and the
 * codec they call (attention/codec.py:91-130); both encodings list the same positions, so the value plane is
 * shared.  A frame whose bitmask does not hold k bits, or whose stream names a position beyond 31 or the same
 * position twice, raises OMMX_ST_BAD_GROUP in *status (optional) and is written as far as it goes.
 */
int ommx_b200_outlier_index_convert(const void *src, void *dst, int64_t frames, int32_t k, int32_t to_relidx7,
                                    int32_t *status, void *stream);

/*
 * Paged decode attention.  Replaces ommx_paged_decode_attention_canonical
 * (ommx_gpu_serve/attention/paged_decode.py:2768-3549): stage 1 = _canonical_splitkv_stage1
 * (:1255), stage 2 = _canonical_lse_merge with the bf16 sink/recent rows fused in (:2366).
 * Writes o / lse in place.  attn_logits is the caller's split workspace
 * f32 [batch, n_q_heads, num_kv_splits+1, head_dim+1] (lane head_dim = log-sum-exp).
 * b_seq_len holds PACKED token counts; split s covers tokens [s*per, min((s+1)*per, seq)) with
 * per = ceil(ceil(seq/num_kv_splits)/32)*32, exactly as the reference.
 */
/*
 * Head-output exchange fused into stage 2, for kv heads sharded over the GPUs of one node (the split vLLM
 * tensor parallelism applies to the reference backend, ommx_gpu_serve/integration/vllm/backend.py:859-873;
 * it stands where that stack runs a collective on the attention output).  Every output element of a rank's
 * stage 2 goes, as one 8-byte word (value, call count), into slot `rank` of every OTHER rank's receive buffer
 * [world, batch, n_q_heads, head_dim] through peer-mapped pointers (plain 8-byte stores over NVLink: a word
 * arrives whole, so no fence and no separate flag; no multicast).  The same thread block then waits for the words
 * of its (sequence, head) row from every peer - their count must equal this call's; about a second of SM clock at
 * most, then OMMX_ST_TIMEOUT - and writes the values to `out`, this rank's plain [world, batch, n_q_heads, head_dim]
 * f32 buffer (its own rows go there directly).  When the call's kernels have finished, `out` holds all ranks' rows.
 * All ranks must make the same sequence of calls on a gather, and consecutive calls must use different receive
 * buffers in turn (a peer may be one call ahead): recv[r] is rank r's buffer for THIS call.  Receive buffers come
 * from ommx_b200_peer_alloc (zero-filled: count 0 is never current); `state` is 2 zero-initialised words of this
 * rank's own memory, shared by all calls of the gather.
 */
typedef struct ommx_head_gather {
    int32_t world, rank;            /* 2..32 ranks */
    uint64_t *const *recv;          /* device array [world]: rank r's receive buffer for this call (recv[rank]: own) */
    float *out;                     /* this rank's [world, batch, n_q_heads, head_dim] f32 result of this call */
    uint32_t *state;                /* this rank's own 2 words (calls made, block ticket), zero at start */
} ommx_head_gather;

typedef struct ommx_decode_args {
    const void *q;                /* bf16 [batch, n_q_heads, head_dim] */
    int32_t q_dtype;              /* OMMX_DT_BF16 */
    int32_t batch, n_q_heads;
    int64_t q_stride_b, q_stride_h;
    ommx_kv_planes planes;
    const void *k_tail, *v_tail;  /* bf16 [batch, T_tail_max, n_kv_heads, head_dim] */
    int64_t tail_stride_b, tail_stride_t, tail_stride_h;
    const int32_t *b_tail_len;    /* [batch] valid residual rows (0 allowed) */
    const int32_t *b_seq_len;     /* [batch] packed tokens */
    const void *req_to_token;     /* [batch, >=pages]  page table */
    const void *req_to_group;     /* [batch, >=groups] group-slot table */
    int32_t table_is_int64;       /* 0: int32 tables, 1: int64 */
    int64_t r2t_stride_b, r2g_stride_b;
    void *o;                      /* [batch, n_q_heads, head_dim] */
    int32_t o_dtype;              /* OMMX_DT_F32 or OMMX_DT_BF16 */
    int64_t o_stride_b, o_stride_h;
    float *lse;                   /* [batch, n_q_heads] */
    int64_t lse_stride_b;
    float *attn_logits;
    int64_t al_stride_b, al_stride_h, al_stride_s;
    int32_t num_kv_splits;
    int32_t max_seq_len;          /* upper bound of b_seq_len (sizes nothing on device; checked) */
    int32_t max_tail_len;
    int32_t seg_group_base;       /* first group of the attended segment (0 = whole sequence) */
    int32_t packed_start_offset;  /* must be 0 */
    float sm_scale, logit_cap;
    int32_t *status;              /* optional */
    int32_t abl_flags;            /* differential-timing ablations (break parity), 0 in service:
                                     1 skip outlier splice, 2 skip V/PV, 4 skip K code dequant, 8 stream only
                                     (reference: OMMX_ABL_* knobs, attention/paged_decode.py:3267-3279);
                                     16 is for tests of the give-up path: stage-1 waits last 2 ms and one ring
                                     fill is announced but not issued, so the call ends with OMMX_ST_TIMEOUT */
    const ommx_head_gather *gather; /* optional: exchange the head outputs with the other ranks in stage 2 */
} ommx_decode_args;

int ommx_b200_decode(const ommx_decode_args *args, void *stream);          /* stage 1 + stage 2 */
int ommx_b200_decode_stage1(const ommx_decode_args *args, void *stream);   /* splits -> attn_logits */
int ommx_b200_decode_stage2(const ommx_decode_args *args, void *stream);   /* attn_logits + tail -> o,lse */

/*
 * ommx_b200_decode with the split workspace taken from a fixed 8 MiB array inside the library
 * instead of args->attn_logits (which is ignored, as are its strides).  This entry point has no
 * counterpart in the reference.  It is for hosts that must not allocate device memory while
 * serving - an engine whose memory pool is frozen after start-up, or a plug-in that receives
 * buffers but no allocator: it calls no cudaMalloc/cudaFree and nothing that allocates.
 * Limit: batch * n_q_heads * num_kv_splits * (head_dim + 1) <= 2 Mi floats, else OMMX_E_ARG.
 * The first call on each device looks up the array's device address (one runtime query, no
 * allocation); make that first call outside any stream capture.  All calls on a device share
 * the one array: two calls that overlap on the GPU (different streams) race; calls ordered on
 * one stream are safe.  Nothing needs clearing between calls - stage 2 reads only the split
 * slots stage 1 of the same call wrote - and the array keeps its last contents otherwise.
 * Every GPU that loads the library holds the 8 MiB until the process exits.
 */
int ommx_b200_decode_static_ws(const ommx_decode_args *args, void *stream);

/*
 * Device-resident decode-step store for a pool of sequences.  Replaces the host loop of
 * MultiSeqKVPool.append_decode_device + decode_inputs_device
 * (ommx_gpu_serve/attention/kv_pool.py:440-488, :1048-1105) and the ring copies
 * _kv_write_token / _kv_gather_tail (attention/kv_store_ops.py:22,42): one call appends one
 * new bf16 K/V row per sequence to its residual ring, quantizes and packs the 32-token group
 * that the step completed (if any) straight from the ring into the sequence's next pages and
 * group slot, advances the device-side sequence lengths, and writes the decode inputs of the
 * step (packed length, residual length, gathered residual rows).  No host synchronisation, a
 * fixed launch shape (CUDA-graph capturable), nothing allocated.
 *
 * A sequence of seq tokens keeps tokens [0, sink) and [boundary, seq) as bf16 rows, with
 * boundary = sink + floor((seq - sink - recent) / 32) * 32 (or min(sink, seq) while seq <= sink +
 * recent), and tokens [sink, boundary) in the planes.  Ring row of token pos:
 * pos < sink ? pos : sink + (pos - sink) % (ring_cap - sink); ring_cap - sink >= recent + 32.
 */
typedef struct ommx_kv_pool {
    ommx_kv_planes planes;            /* pooled planes of all sequences */
    void *k_hist, *v_hist;            /* bf16 [num_seqs, ring_cap, n_kv_heads, head_dim] */
    int32_t num_seqs, ring_cap;
    int32_t sink_tokens, recent_window;
    int32_t *seq_len;                 /* device int32 [num_seqs]: tokens held, advanced by the call */
    const int32_t *req_to_token;      /* device int32 [num_seqs, pages_per_seq] page ids */
    const int32_t *req_to_group;      /* device int32 [num_seqs, groups_per_seq] group slots */
    int32_t pages_per_seq, groups_per_seq;
} ommx_kv_pool;

typedef struct ommx_kv_append_args {
    ommx_kv_pool pool;
    const void *k_new, *v_new;        /* bf16 [batch, n_kv_heads, head_dim]; NULL with advance = 0 */
    int64_t new_stride_b, new_stride_h;
    const void *slots;                /* device [batch]: pool slot of each row, NULL = 0..batch-1 */
    int32_t batch;
    int32_t advance;                  /* 1: append + pack + advance; 0: only (re)build the decode inputs;
                                         2: append + pack, pool.seq_len left alone (the caller advances it) */
    int32_t outlier_select, use_pow2; /* as in ommx_pack_args; outlier_select must be 1 (signed) */
    void *k_tail, *v_tail;            /* out, optional: bf16 [batch, max_tail, n_kv_heads, head_dim] */
    int32_t max_tail;
    int32_t *b_seq_len, *b_tail_len;  /* out, optional: device int32 [batch] */
    int32_t *status;                  /* optional */
    const void *write_pos;            /* optional, device [batch]: tokens each row's sequence holds before this
                                         step (the absolute position the new row is written at), instead of
                                         pool.seq_len[slot]; with advance = 1 seq_len[slot] becomes write_pos + 1.
                                         This is the (rows, cols) form of MultiSeqKVPool.append_decode_captured
                                         (attention/kv_pool.py:490-524) and CanonicalKVStore.write_token
                                         (attention/kv_store.py:361-385). */
    int32_t index_is_int64;           /* slots and write_pos hold int64 (else int32) */
} ommx_kv_append_args;

int ommx_b200_kv_append_decode(const ommx_kv_append_args *args, void *stream);

/*
 * Residual rows by absolute token position: k_tail/v_tail[i, y] = ring row of token tail_idx[i, y] of
 * sequence slot sel[i] (NULL: slot i).  Replaces _kv_gather_tail (attention/kv_store_ops.py:42-57) as
 * called by CanonicalKVStore.gather_tail_into (attention/kv_store.py:397-427) and
 * MultiSeqKVPool.decode_inputs_captured (attention/kv_pool.py:886-936).  sel and tail_idx are device
 * int32 or int64; k_tail/v_tail are bf16 [batch, rows, n_kv_heads, head_dim], contiguous.  Only
 * pool->k_hist, v_hist, ring_cap, sink_tokens, num_seqs and the head geometry are read.  A negative
 * position or a slot outside the pool zero-fills the row and sets a status bit.
 */
int ommx_b200_kv_gather_tail(const ommx_kv_pool *pool, const void *sel, const void *tail_idx,
                             int32_t index_is_int64, int32_t batch, int32_t rows,
                             void *k_tail, void *v_tail, int32_t *status, void *stream);

/*
 * Split count this library prefers for (max context, batch, local kv heads) on the current
 * device.  Replaces _auto_num_kv_splits (attention/paged_decode.py:409-461), which callers
 * use to size attn_logits once.
 */
/*
 * Device memory that other processes of the node can map (CUDA IPC), for ommx_head_gather.  `alloc` returns a
 * zero-filled allocation and its 64-byte handle; `open` maps another process's allocation into this one (peer
 * access over NVLink) and `close` unmaps it; `free` releases an own allocation.  Call them outside stream capture.
 */
int ommx_b200_peer_alloc(size_t bytes, void **ptr, void *handle64);
int ommx_b200_peer_open(const void *handle64, void **ptr);
int ommx_b200_peer_close(void *ptr);
int ommx_b200_peer_free(void *ptr);

int ommx_b200_auto_num_kv_splits(int32_t max_seq_len, int32_t batch, int32_t n_kv_heads);
/* Smallest split count ommx_b200_decode accepts for a context of max_seq_len packed tokens. */
int ommx_b200_min_num_kv_splits(int32_t max_seq_len, int32_t page_size);

/*
 * Merge P partial softmax states over disjoint KV segments.  Replaces merge_attention_states
 * (attention/paged_decode.py:3556-3624, kernel :2650-2690).
 * o_parts f32 [P, R, D], lse_parts f32 [P, R], valid_lens int32 [R] or NULL (all P valid).
 */
int ommx_b200_merge_states(const float *o_parts, const float *lse_parts, const int32_t *valid_lens,
                           int32_t P, int32_t R, int32_t D, float *o, float *lse, void *stream);

/* Host-side twins of the two table-driven decisions inside the packer (no GPU needed):
 * round_half_even(log2(x)) for x > 0, and the FP4 E2M1 code of m
 * (reference: attention/pack.py:459-463, attention/codec.py:45-65). */
int ommx_b200_host_pow2_exponent(float x);
int ommx_b200_host_fp4_encode(float m);

int ommx_b200_abi_version(void);
const char *ommx_b200_last_error(void);   /* thread-local text of the last negative return */
/* Kernels launched by this library since load (or since the last reset), for launch evidence;
 * mirrors launch_stats()/reset_launch_stats() (attention/paged_decode.py:2728-2739). */
int64_t ommx_b200_launch_count(void);
void ommx_b200_reset_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* OMMX_B200_H_ */
