/*
 * hqmq_b200 -- C ABI of the B200 (sm_100a) kernels for the HQMQ KV-cache hot path:
 * encode (chunk norm, Med3x flag, per-token-max radius code, nearest codeword of the
 * 24*S product codebook), packed dequant, and fused decode attention over the compressed
 * cache.  Everything the Python host layer does on a GPU goes through these entry points.
 *
 * Conventions
 *   - every function returns 0 on success or a negative HQMQ_ERR_* code; nothing throws,
 *     prints or exits.  hqmq_strerror() names a code.
 *   - the caller owns every buffer (device pointers unless stated otherwise); the library
 *     allocates no device memory and keeps no pointer after returning.
 *   - all work is enqueued on the given CUDA stream (a cudaStream_t passed as void*);
 *     nothing synchronises.  Argument problems are detected on the host before any launch.
 *   - structs start with struct_size = sizeof(the struct) so that layouts can grow.
 *
 * The interfaces these replace live in the reference repository (kswain98/hqmq); each
 * declaration cites them as path:line.
 */
#ifndef HQMQ_B200_H
#define HQMQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HQMQ_ABI_VERSION 4

/* error codes */
#define HQMQ_OK 0
#define HQMQ_ERR_ARG (-1)         /* null pointer, bad struct_size, bad enum */
#define HQMQ_ERR_SHAPE (-2)       /* d % 4, H_q % H_kv, sizes out of the supported range */
#define HQMQ_ERR_DTYPE (-3)
#define HQMQ_ERR_ALIGN (-4)       /* pointer or stride not aligned as documented */
#define HQMQ_ERR_WORKSPACE (-5)   /* workspace missing or too small */
#define HQMQ_ERR_ARCH (-6)        /* device is not compute capability 10.x */
#define HQMQ_ERR_CUDA (-7)        /* a CUDA runtime call failed (launch configuration etc.) */
#define HQMQ_ERR_UNSUPPORTED (-8)
#define HQMQ_ERR_CAPACITY (-9)    /* packed cache or outlier side buffer too small */
#define HQMQ_ERR_STATIC_SCRATCH (-10) /* needs more scratch than the library's built-in buffer holds */
#define HQMQ_ERR_TIMEOUT (-11)    /* a bounded device-side wait ran out (reported by the host layer from a status word) */

/* element types */
#define HQMQ_F32 0
#define HQMQ_F16 1
#define HQMQ_BF16 2
#define HQMQ_I32 3
#define HQMQ_I16 4
#define HQMQ_I8 5
#define HQMQ_U8 6
#define HQMQ_I64 7

/* Tokens per outlier-offset block of the native layout (= the attention kernel's KV tile). */
#define HQMQ_OUT_BLOCK 16
/* Plane capacities (T_cap) are multiples of this many tokens. */
#define HQMQ_T_ALIGN 64
/* Size of one record of the optional `ofrag` plane, and the most records a tile may own. */
#define HQMQ_OFRAG_BYTES 528
#define HQMQ_OFRAG_MAX_PER_TILE 2

/*
 * Native compressed layout of one K or V tensor (what the roofline is measured on).
 * The reference has no in-memory compressed format: its packed tuple is int32 indices +
 * integer radius codes + per-token scale (src/quantizers/hqmq_attention.py:11-18) and
 * its outlier wrapper keeps dense tensors (src/quantizers/outlier_aware.py:86).
 *
 * Per (batch b, KV head h) there are four token-major planes of capacity T_cap tokens
 * (T_cap a multiple of 64):
 *   codes  [B][H][T_cap][row_bytes]  one bit-packed row per token; chunk c occupies bits
 *          [c*cb, (c+1)*cb) of the row, little-endian, cb = idx_bits + radius_bits,
 *          field = native_idx | (rq << idx_bits), idx_bits = ceil(log2(24*S)).
 *          native_idx = ((a*S + s) << 3) | u where the reference's primary index p
 *          (src/quantizers/spherical.py:22-43) is factored as p = u * omega^a with u one
 *          of the 8 axis units (reference order 0..7) and omega = (1+i+j+k)/2;
 *          hqmq_native_index_maps() gives both directions.  row_bytes is a multiple of 4.
 *   rs     [B][H][T_cap]             per-token radius scale r_max: fp16 / bf16 bits (2 B per
 *          token, what the byte accounting assumes) or fp32 (exact fake-quant round trips)
 *   flags  [B][H][T_cap]             uint32, bit c set = chunk c is an outlier kept in
 *          full precision (NULL when the tensor was encoded without Med3x); the radius code
 *          stored in the row for a flagged chunk is 0 (the reference would compute one, but its
 *          wrapper discards the quantised value of a flagged chunk: outlier_aware.py:86)
 *   out_vals [B][H][out_cap][4]      the original 4 values of every flagged chunk as
 *          fp16 / bf16 / fp32, in (token, chunk) order
 *   out_off  [B][H][T_cap/16 + 1]    number of flagged chunks before each 16-token block
 *   out_count[B][H]                  flagged chunks stored so far
 * Appending tokens never rewrites an earlier row.
 *
 * Optional acceleration plane for a K tensor with outliers (no counterpart in the reference; derived
 * data, never needed to reconstruct the tensor):
 *   ofrag    [B][H][ofrag_cap][528]  records that hold the flagged chunks of one 16-token block in
 *          the operand order of the attention kernel's tensor-core instruction, so that their
 *          scores cost one shared-memory load and one MMA.  A record covers up to four distinct
 *          chunk positions c_0..c_3 flagged anywhere in the block: bytes 0..3 = c_0..c_3
 *          (0xFF = unused), bytes 4..15 = 0, then 32 entries of 16 bytes; entry l (row r = l/4,
 *          position j = l%4) holds eight fp16 values v(r,0) v(r,1) v(r+8,0) v(r+8,1) v(r,2) v(r,3)
 *          v(r+8,2) v(r+8,3) with v(t,e) = x[token t of the block][4*c_j + e] * qmax / rs[t] if
 *          chunk c_j of token t is flagged, else 0.
 *   ofrag_off[B][H][T_cap/16 + 1]    records before each 16-token block.  hqmq_encode writes a
 *          block's records in the call that completes the block (its 16th token), from the flag
 *          words and out_vals, if the block has at most 4*HQMQ_OFRAG_MAX_PER_TILE distinct flagged
 *          positions and the records fit ofrag_cap; every other block (the last, incomplete one
 *          included) owns no record and the attention kernels take its outliers from flags/out_vals.
 */
typedef struct hqmq_packed {
  uint32_t struct_size;
  int32_t B, H;
  int32_t T_cap;        /* plane capacity in tokens, multiple of 64 */
  int32_t n_chunks;     /* d_head / 4, 1..32 */
  int32_t S;            /* secondary codebook size, 24*S <= 65536 */
  int32_t radius_bits;  /* 1..8 */
  int32_t row_bytes;    /* hqmq_row_bytes(n_chunks, S, radius_bits) */
  int32_t scale_dtype;  /* HQMQ_F16, HQMQ_BF16 or HQMQ_F32: element type of rs */
  int32_t out_dtype;    /* HQMQ_F16, HQMQ_BF16 or HQMQ_F32: element type of out_vals */
  int32_t out_cap;      /* capacity of out_vals per (b,h), in chunks */
  int32_t ofrag_cap;    /* capacity of ofrag per (b,h), in records (0 when ofrag is NULL) */
  uint8_t* codes;
  void* rs;
  uint32_t* flags;
  void* out_vals;
  uint32_t* out_off;
  uint32_t* out_count;
  uint8_t* ofrag;       /* NULL = no fragment records; 16-byte aligned */
  uint32_t* ofrag_off;
} hqmq_packed;

/*
 * The reference's packed tuple (src/quantizers/hqmq_attention.py:11-18): idx and rq are
 * (B,H,T,n_chunks) with unit stride on the last dim, rs is (B,H,T); strides in elements.
 */
typedef struct hqmq_ref_packed {
  uint32_t struct_size;
  int32_t idx_dtype;    /* HQMQ_I32 or HQMQ_I64 or HQMQ_I16 */
  int32_t rq_dtype;     /* HQMQ_I32, HQMQ_I16, HQMQ_I8, HQMQ_U8, HQMQ_I64 */
  int32_t rs_dtype;     /* HQMQ_F32, HQMQ_F16, HQMQ_BF16 */
  const void* idx;
  const void* rq;
  const void* rs;
  int64_t idx_stride[3]; /* b, h, t */
  int64_t rq_stride[3];
  int64_t rs_stride[2];  /* b, h (t has unit stride) */
} hqmq_ref_packed;

/* ---- library ------------------------------------------------------------------------ */
int hqmq_abi_version(void);
const char* hqmq_strerror(int code);
/* HQMQ_OK if `device` has compute capability 10.x, else HQMQ_ERR_ARCH. */
int hqmq_device_check(int device);
int hqmq_idx_bits(int S);
int hqmq_row_bytes(int n_chunks, int S, int radius_bits);
/* Host tables, 24 entries each: ref_to_native[p] = (a << 3) | u, native_to_ref[(a << 3) | u] = p. */
int hqmq_native_index_maps(uint8_t* ref_to_native, uint8_t* native_to_ref);

/* ---- codebook ----------------------------------------------------------------------- */
/*
 * Derive the device tables the kernels use from the reference-order joint table
 * joint[H][24*S][4] (fp32, k = p*S + s; src/quantizers/hqmq.py:119-143):
 *   table16[H][24*S][4] fp16 in NATIVE index order (gathered by the attention/dequant kernels).
 */
int hqmq_codebook_tables(const float* joint, int H, int S, uint16_t* table16, void* stream);

/* ---- encode --------------------------------------------------------------------------- */
/*
 * Nearest-codeword look-up table of one joint codebook (H heads).  A direction is folded by its nearest Hurwitz
 * unit (the codebook is invariant under the 24 units), which leaves an octahedron of folded directions; a grid over
 * it names, per cell, every codeword that can win somewhere in the cell -- a single one for almost half of the
 * cells, two on average.  It turns the reference's exhaustive argmax over 24*S similarities
 * (src/quantizers/hqmq.py:158,164) into zero to four dot products per chunk with the same result.  Build once per
 * (layer, K|V) codebook.  hqmq_encode_lut_build picks the finest grid whose tables fit the encoder's shared memory
 * next to the codebook and synchronises the stream to do so.  hqmq_encode_lut_footprint synchronises the stream and
 * returns the shared-memory bytes of the largest head's table (-1 if the codebook got no table: the encoder then
 * searches exhaustively); pass it on in hqmq_encode_args.lut_footprint.
 */
size_t hqmq_encode_lut_bytes(int H, int S);
size_t hqmq_encode_lut_workspace_bytes(int H, int S);
int hqmq_encode_lut_build(const float* joint, int H, int S, void* lut, size_t lut_bytes, void* workspace,
                          size_t workspace_bytes, void* stream);
int hqmq_encode_lut_footprint(const void* lut, int H, int* footprint, void* stream);

typedef struct hqmq_encode_args {
  uint32_t struct_size;
  int32_t x_dtype;          /* HQMQ_F32 / HQMQ_F16 / HQMQ_BF16 */
  const void* x;            /* (B,H,T_new,d), last dim contiguous */
  int64_t x_stride[3];      /* b, h, t in elements */
  int32_t T_new;            /* tokens in this call */
  int32_t t_start;          /* row of the packed planes that receives token 0 of x */
  const float* qs;          /* (H,S,4) unit secondary quaternions, fp32 */
  const float* joint;       /* (H,24*S,4) fp32 joint table, reference order */
  float median_mult;        /* multiplier C of the threshold statistic (Med3x: 3); <= 0 disables outlier flagging */
  int32_t search;           /* 0 = default (look-up table when `lut` is given), 1 = exhaustive scan over the S secondaries */
  hqmq_packed dst;          /* destination planes */
  float* med_out;           /* optional (H,) fp32: the per-head median of this call */
  const void* lut;          /* optional nearest-codeword table of this codebook (hqmq_encode_lut_build) */
  int32_t lut_footprint;    /* hqmq_encode_lut_footprint() of `lut` (0 = unknown, assume the capacity) */
  float quantile;           /* 0: the threshold is median_mult x the per-head median (Med3x).  q in (0, 1): median_mult x
                               torch.quantile(norms, q) per head, with torch's rank arithmetic and interpolation (the
                               reference wrapper's threshold_mode="fraction": q = 1 - fraction, median_mult = 1) */
  const float* med_in;      /* optional (H,) fp32, device: per-head medians to use instead of this call's own; for a
                               head whose batch entries are spread over several GPUs (hqmq_med3x_hist / _select) */
} hqmq_encode_args;

/*
 * Replaces HQMQQuantizer._qdq (src/quantizers/hqmq.py:145-216, unit-magnitude linear
 * radius path) and OutlierAwareHQMQQuantizer._qdq (src/quantizers/outlier_aware.py:56-87,
 * threshold_mode="median_mult"), emitting the compressed representation instead of a
 * dense fake-quantised tensor.  The Med3x median is taken over all B*T_new*n_chunks chunk
 * norms of each head of THIS call, like the reference.
 */
size_t hqmq_encode_workspace_bytes(const hqmq_encode_args* args);
int hqmq_encode(const hqmq_encode_args* args, void* workspace, size_t workspace_bytes, void* stream);

/*
 * The K and the V tensor of one layer in one call: the reference cache quantises both on every update
 * (src/model_utils.py:29-32, QuantizedCache.update).  Same results as hqmq_encode(k) followed by
 * hqmq_encode(v); each tensor keeps its own median, tables and planes.  For the decode-time append (a small
 * call, the same batch / heads / new tokens / head dim for both tensors) the whole append -- codes, scales, flags,
 * offset scan and side planes of both tensors -- is ONE kernel launch after a memset of the two status words (a
 * single-tensor small call takes three launches); other shapes run one tensor after the other.  The workspace holds K's part
 * first and V's part at the next multiple of 256 bytes; the first word of each part is that tensor's status
 * word (hqmq_read_status on workspace, and on workspace + round_up(hqmq_encode_workspace_bytes(k), 256)).
 */
size_t hqmq_encode_pair_workspace_bytes(const hqmq_encode_args* k, const hqmq_encode_args* v);
int hqmq_encode_pair(const hqmq_encode_args* k, const hqmq_encode_args* v, void* workspace, size_t workspace_bytes,
                     void* stream);

/*
 * Med3x median of heads whose batch entries live on SEVERAL GPUs.  The reference takes the median over every
 * batch entry of a head in one call (src/quantizers/outlier_aware.py:63-72); when the batch of a head is
 * partitioned across GPUs, the same number comes from a three-level radix select whose histograms are summed
 * across those GPUs between the levels (integer sums, so every GPU derives identical bits):
 *     for level in 0, 1, 2:
 *         hqmq_med3x_hist(args, level, state, ...)        -- histogram of this GPU's chunk norms (level 0 clears state)
 *         sum the 2 * 2048 uint32 words at  state + ((h * 3 + level) * 2 * 2048) * 4  of every head h over the GPUs
 *                                                        (ncclAllReduce; a sum over the whole histogram area is as good)
 *         hqmq_med3x_select(H, level, n_total, C, state, ..., med_out)   -- n_total = chunk norms per head over all GPUs
 *     hqmq_encode(args with med_in = med_out, ...)
 * `state` is hqmq_med3x_state_bytes(H) bytes of device memory, 16-byte aligned, owned by the caller.  `args` is
 * the struct of the hqmq_encode call that follows and is validated like it; hqmq_med3x_hist reads x and the
 * geometry only and writes nothing but `state`.  A GPU that holds no token of the heads (T_new = 0) still takes
 * part in the sums.  The reference has no multi-GPU path; these have no counterpart there.
 */
size_t hqmq_med3x_state_bytes(int H);
int hqmq_med3x_hist(const hqmq_encode_args* args, int level, void* state, size_t state_bytes, void* stream);
int hqmq_med3x_select(int H, int level, uint64_t n_total, float median_mult, void* state, size_t state_bytes,
                      float* med_out, void* stream);
/*
 * Device-detected problems are recorded in the first word of the workspace a call was given, never
 * printed or trapped on.  This copies that word to the host after synchronising `stream`.
 *   workspace of hqmq_encode:       bit 0 = the outlier side buffer (out_cap) was too small; rows,
 *                                   flags and counts are complete, payload entries beyond the
 *                                   capacity were dropped
 *   workspace of hqmq_attn_decode:  non-zero = some call on this workspace gave up on a bounded wait
 *                                   for a staged copy; the output rows of that call are not valid (NaN where
 *                                   a merge still ran, untouched elsewhere)
 * No counterpart in the reference (its kernels have no device-side status).
 */
int hqmq_read_status(const void* workspace, uint32_t* status, void* stream);

/* ---- layout conversion ---------------------------------------------------------------- */
/*
 * native -> reference tuple for tokens [t0, t0+T): idx int32 (B,H,T,n) in reference order,
 * rq int32 (B,H,T,n), rs fp32 (B,H,T), flags uint8 (B,H,T,n) (may be NULL), all contiguous.
 */
int hqmq_unpack(const hqmq_packed* src, int t0, int T, int32_t* idx, int32_t* rq, float* rs,
                uint8_t* flags, void* stream);
/* reference tuple -> native planes at rows [t_start, t_start+T); indices are reference order. */
int hqmq_pack(const hqmq_ref_packed* src, int T, hqmq_packed* dst, int t_start, void* stream);

/* ---- dequant -------------------------------------------------------------------------- */
typedef struct hqmq_dequant_args {
  uint32_t struct_size;
  int32_t layout;            /* 0 = native (src_native, table16 native order), 1 = reference tuple */
  hqmq_packed src_native;
  hqmq_ref_packed src_ref;
  int32_t B, H, T, n_chunks; /* reference layout only (native takes them from src_native) */
  int32_t t0;                /* first token (native layout) */
  int32_t r_qmax;
  int32_t scale_first;       /* 0: cw*((rq*rs)/qmax) as hqmq_attention.py:61; 1: cw*(rq*(rs/qmax)) as hqmq.py:210-216 */
  int32_t joint_dtype;       /* reference layout: dtype of `joint` (arithmetic is done in it) */
  const void* joint;         /* reference layout: (H,K,4), reference order */
  int32_t K;                 /* reference layout: rows of joint per head */
  const float* joint_f32;    /* native layout: (H,24S,4) fp32 reference order */
  int32_t out_dtype;
  void* out;                 /* (B,H,T,4*n_chunks) contiguous */
  int32_t merge_outliers;    /* native layout with flags: write the original values of flagged chunks */
} hqmq_dequant_args;

/*
 * Replaces _decode_kv_torch (src/quantizers/hqmq_attention.py:39-65) and
 * hqmq_decode_triton (src/quantizers/hqmq_kernel.py:102-132).
 */
int hqmq_dequant(const hqmq_dequant_args* args, void* stream);

/* ---- decode attention ------------------------------------------------------------------ */
typedef struct hqmq_attn_args {
  uint32_t struct_size;
  int32_t layout;            /* 0 = native, 1 = reference tuple */
  int32_t q_dtype;           /* element type of Q */
  int32_t o_dtype;           /* element type of O (may differ from Q, e.g. fp32 output for bf16 queries) */
  const void* Q;             /* (B,H_q,T_q,d) */
  int64_t q_stride[3];       /* b, h, t in elements; last dim contiguous */
  void* O;                   /* (B,H_q,T_q,d) */
  int64_t o_stride[3];
  int32_t B, H_q, H_kv, T_q, T_kv, d;
  int32_t r_qmax;
  int32_t causal;            /* 0: none.  1: top-left aligned, query i sees keys 0..i (hqmq_attention.py:100,229).
                                2: bottom-right aligned, query i sees keys 0..T_kv - T_q + i (the queries are the
                                last T_q positions of a cache that already holds them: a prompt chunk) */
  int32_t window;            /* > 0: only the last `window` keys (sliding window); 0 = all */
  float softmax_scale;       /* <= 0: 1/sqrt(d) */
  int32_t kv_splits;         /* 0 = choose; n > 0 = split the key range into n pieces */
  int32_t partials_only;     /* 1: leave (m,l,o) partials of ONE piece per (b,h_q) in `partials` (sequence-parallel use) */
  /* native layout */
  hqmq_packed K, V;
  const uint16_t* table_K;   /* (H_kv,24S,4) fp16 native order (hqmq_codebook_tables) */
  const uint16_t* table_V;
  /* reference layout */
  hqmq_ref_packed K_ref, V_ref;
  int32_t joint_dtype;
  int32_t K_size;            /* rows per head of joint_K / joint_V */
  const void* joint_K;       /* (H_kv,K,4) */
  const void* joint_V;
  float* partials;           /* partials_only: (B,H_q,T_q,d+2) fp32: o[d], m, l */
} hqmq_attn_args;

/*
 * Replaces fused_hqmq_attention_triton (src/quantizers/hqmq_attention.py:425-518; kernel
 * :120-265) with the semantics of its oracle fused_hqmq_attention_torch (:68-101).
 */
size_t hqmq_attn_workspace_bytes(const hqmq_attn_args* args);
int hqmq_attn_decode(const hqmq_attn_args* args, void* workspace, size_t workspace_bytes, void* stream);

/*
 * hqmq_attn_decode for hosts that cannot provide a workspace.  No counterpart in the reference.
 *
 * Who needs it: a process that has no device allocator to call -- an inference server that handed all free
 * HBM to its cache pool when it started, so that any later cudaMalloc fails, or a binding from another
 * language that wraps only this header.  The scratch that hqmq_attn_decode takes from the caller (the
 * per-warp partial results) is here a fixed buffer of HQMQ_ATTN_STATIC_SCRATCH_BYTES inside the library
 * itself; each GPU that loads the library carries that much until the process ends.  The function calls
 * no cudaMalloc / cudaFree and no allocating library routine; Q, O and the cache planes are still the
 * caller's.
 *
 *   - A problem whose partials do not fit (hqmq_attn_workspace_bytes(args) > HQMQ_ATTN_STATIC_SCRATCH_BYTES)
 *     is rejected with HQMQ_ERR_STATIC_SCRATCH before anything is launched; use hqmq_attn_decode then.
 *   - The first call on a device looks up the buffer's device address (cudaGetSymbolAddress) with that
 *     device current, and caches it; make that first call during set-up, before any stream capture begins.
 *     Call it with the device current that owns `stream`.
 *   - All calls on a device share the one buffer, and it keeps what the previous call left.  Nothing in it
 *     needs clearing between calls (every value read was written by the same call), but two calls that
 *     overlap on the GPU -- different streams, or graphs replayed concurrently -- race on it: serialise them.
 *   - The one word that must start at zero, the give-up word of the bounded waits, is cleared on `stream`
 *     at the start of every call.  hqmq_attn_static_status() synchronises `stream` and returns that word of
 *     the current device's buffer: non-zero = the most recent call on this device gave up on a bounded wait
 *     for a staged copy and its output rows are NaN (the same meaning hqmq_read_status has for a caller's
 *     workspace).  Call it with the same device current.
 */
#define HQMQ_ATTN_STATIC_SCRATCH_BYTES (16u << 20)
int hqmq_attn_decode_static(const hqmq_attn_args* args, void* stream);
int hqmq_attn_static_status(uint32_t* status, void* stream);

/*
 * Merge n_parts partial results (o[d], m, l per row, as written with partials_only; m is the maximum
 * of score * log2(e)) into normalised outputs.  parts is (rows, n_parts, d+2) fp32, or with
 * part_major != 0 (n_parts, rows, d+2): the layout an all_gather of per-GPU partials produces.  out is
 * (rows, d) of out_dtype.  No counterpart in the reference (it has no split-KV or multi-GPU path).
 */
int hqmq_combine_partials(const float* parts, int n_parts, int64_t rows, int d, int part_major, int out_dtype,
                          void* out, void* stream);

/* ---- exchange of sequence-split partials over NVLink by direct stores ------------------------------------ */
/*
 * For one long context split by sequence over `world` GPUs (one process each): instead of an all_gather of
 * the per-GPU partial blocks (partials_only output of hqmq_attn_decode, rows * (d + 2) floats), every rank
 * stores its block into slot `rank` of every peer's receive buffer through peer-mapped pointers and then
 * publishes the step's epoch in the peer's flag words; the receiver waits on its OWN memory only.  No
 * counterpart in the reference (it is single-GPU).
 *
 *   recv[p]   address, in THIS process, of rank p's receive buffer: float[2][world][block_floats]
 *             (hqmq_exchange_recv_bytes; 16-byte aligned; two halves used alternately by epoch parity, so a
 *             rank that is one step ahead never overwrites a block that is still being merged)
 *   flags[p]  address, in this process, of rank p's flag words: uint32[2][world], zero before first use
 *   recv[rank] / flags[rank] are this rank's own buffers; the others are the peers' (cudaIpc or any other
 *   peer mapping; peer access must be enabled: hqmq_exchange_enable_peer).  block_floats must be a multiple of 4.
 *
 * Per step, with epoch = 1, 2, 3, ... (the same on every rank, never 0), on the rank's stream:
 *     hqmq_attn_decode(partials_only = 1)                      -> local block
 *     hqmq_exchange_push(x, local, epoch, stream)              -> stores into all world receive buffers
 *     hqmq_exchange_wait(x, epoch, max_polls, status, stream)  -> returns on the GPU when every rank's epoch
 *                                                                 word arrived, or after max_polls polls
 *                                                                 (0 = default, about a second): then bit r of
 *                                                                 *status (device uint32, caller-zeroed) is set
 *                                                                 for every rank r whose block is missing
 *     hqmq_combine_partials(recv[rank] + (epoch & 1) * world * block_floats, world, rows, d, 1, ...)
 * A non-zero status after synchronising means the output of that step is invalid (HQMQ_ERR_TIMEOUT in the
 * host layer); nothing hangs.  The kernels of one GPU never wait for each other; do not run two ranks of one
 * exchange on the same GPU concurrently.
 */
#define HQMQ_EXCHANGE_MAX_RANKS 16
typedef struct hqmq_exchange {
  uint32_t struct_size;
  int32_t world, rank;
  int32_t reserved;
  int64_t block_floats;
  float* recv[HQMQ_EXCHANGE_MAX_RANKS];
  uint32_t* flags[HQMQ_EXCHANGE_MAX_RANKS];
} hqmq_exchange;
/* Lets kernels of the CURRENT device store into memory that lives on `peer_device` (cudaDeviceEnablePeerAccess;
 * an IPC mapping opened with the peer's device current does not enable it by itself).  Once per peer, at set-up. */
int hqmq_exchange_enable_peer(int peer_device);
/* Mapping the peers' buffers (one process per GPU).  export: the 64-byte CUDA IPC handle of the allocation that
 * holds `ptr`, and ptr's byte offset in it; send both to the peers by any host channel.  open: map a peer's
 * allocation for stores from the CURRENT device (open it with the device current whose kernels will store into
 * it -- a mapping opened with the buffer's own device current is not reachable from another device); the
 * buffer is at base + offset.  One open per handle and process; close after a barrier, at tear-down. */
#define HQMQ_IPC_HANDLE_BYTES 64
int hqmq_exchange_ipc_export(const void* ptr, unsigned char* handle64, int64_t* offset);
int hqmq_exchange_ipc_open(const unsigned char* handle64, void** base_out);
int hqmq_exchange_ipc_close(void* base);
/* Set-up check, once: every address of `x` is device memory known to this process, the own buffers live on the
 * current device, and peer access to every other buffer's device is (made) enabled. */
int hqmq_exchange_verify(const hqmq_exchange* x);
size_t hqmq_exchange_recv_bytes(int world, int64_t block_floats);
size_t hqmq_exchange_flag_bytes(int world);
int hqmq_exchange_push(const hqmq_exchange* x, const float* local, uint32_t epoch, void* stream);
int hqmq_exchange_wait(const hqmq_exchange* x, uint32_t epoch, uint32_t max_polls, uint32_t* status, void* stream);
/* push + wait + hqmq_combine_partials(part_major) of one step in ONE launch: `local` (rows x (d + 2) fp32) goes to every
 * rank, the blocks of all ranks are awaited (same bound, same status word as hqmq_exchange_wait) and merged into
 * out (rows x d, out_dtype).  rows + world <= 1184 (HQMQ_ERR_UNSUPPORTED beyond: use the three calls).  Two such
 * launches that wait for EACH OTHER must not share one GPU (ranks are GPUs). */
int hqmq_exchange_step(const hqmq_exchange* x, const float* local, uint32_t epoch, uint32_t max_polls, uint32_t* status,
                       int64_t rows, int d, int out_dtype, void* out, void* stream);
#ifdef __cplusplus
}
#endif
#endif /* HQMQ_B200_H */
