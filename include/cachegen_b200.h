/*
 * cachegen_b200 -- C ABI of the B200-native CacheGen KV-cache codec.
 *
 * One shared library (libcachegen_b200.so, sm_100a) exports exactly the calls a
 * binding for the reference's codec path needs: the four `torchac_cuda` entry
 * points (LMCache/third_party/torchac_cuda/main.cpp:14-17 in the reference) and
 * the fused calls that replace the chains of torch ops around them in
 * LMCache/lmcache/storage_backend/serde/cachegen_{encoder,decoder}.py.
 *
 * Conventions
 *  - plain pointers and sizes only; every pointer is a DEVICE pointer unless its
 *    name ends in `_host`; `stream` is a cudaStream_t passed as void* (NULL =
 *    the legacy default stream);
 *  - a call only enqueues work on `stream` and returns; results are valid after
 *    the stream is synchronised; nothing is allocated, the caller owns all memory;
 *  - return value: 0 = enqueued, < 0 = rejected argument (CG_E_*), nothing was
 *    launched.  Conditions only the GPU can see (a stream that outgrew its
 *    scratch row, lengths that do not add up) are OR-ed into the caller's
 *    `status` word (int32 in device memory, may be NULL) as CG_S_* bits;
 *  - strides are in ELEMENTS of the array they describe;
 *  - 16-bit float type codes: CG_F16 = 0, CG_BF16 = 1;
 *  - a "row" is one of the NL = 2*L rows of the codec's working tensors: the L
 *    key layers followed by the L value layers (torch.cat((new_key, new_value)),
 *    cachegen_encoder.py:263);
 *  - a "stream" is the arithmetic-coded bitstream of one (row, channel) over the
 *    <= CG_MAX_TOKENS_PER_STREAM tokens of one sub-chunk.
 */
#ifndef CACHEGEN_B200_H
#define CACHEGEN_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CG_F16 0
#define CG_BF16 1

/* cachegen_basics.py:8 CACHEGEN_GPU_MAX_TOKENS_PER_CHUNK; torchac_kernel_enc_new.cu:10 */
#define CG_MAX_TOKENS_PER_STREAM 256
/* torchac_kernel_dec_new.cu:6 MAX_LP (the encoder's limit is 48, torchac_kernel_enc_new.cu:6) */
#define CG_MAX_LP 64
/* worst-case stream length for n tokens: 16 bits per symbol plus the flush */
#define CG_STREAM_CAPACITY(ntokens) (2 * (ntokens) + 8)
/* channels of one row handled by one thread block (one thread per stream) */
#define CG_GROUP_CHANNELS 128
/* sub-chunks one fused decode launch can take */
#define CG_MAX_DECODE_JOBS 40

/* Table kinds of cg_decode_job.tables.
 * CG_TABLES_CDF:    int16 [nrows, nchannels, lp], the reference's tables (calculate_cdf).
 * CG_TABLES_COUNTS: the histograms the tables are built from, one byte per (row, non-centre symbol,
 *   channel): row r has 2*Cq_r stored symbols (Cq_r = bins_r // 2 - 1; symbols 0..2*Cq_r except the
 *   centre symbol Cq_r, whose count is the chunk's token count minus the others), laid out as
 *   counts[table_row_off[r] + j * nchannels + channel], j = symbol index with the centre skipped,
 *   table_row_off[r] = nchannels * sum of 2*Cq over the rows before r.  The decoder rebuilds
 *   cdf[i] = (uint16)((0xFFFF - max_bins) * #{sym < i} / ntokens) + i from them (cal_cdf.cu:11-15,40-49):
 *   a table costs 14 or 30 bytes instead of 66.  Usable when no non-centre count exceeds 255.
 * CG_TABLES_SPARSE: the same byte counts with the zero counts left out (cg_pack_sparse_tables writes
 *   it).  `tables` holds three parts, each starting on a 16-byte boundary:
 *     group_off  uint32 [nrows * G + 1], G = ceil(nchannels / 128): where each (row, 128-channel
 *                group)'s counts start inside `counts`; the last entry is the size of `counts`
 *     masks      per (row, channel) one bit per non-centre symbol that has a non-zero count, bit j =
 *                stored symbol j as above; uint16 for rows with 2*Cq_r <= 16, else uint32; row r
 *                starts table_row_off[r] bytes into the part and table_row_off[nrows] is its size
 *     counts     the non-zero counts, one byte each: groups in (row, group) order, inside a group
 *                channel after channel, inside a channel by rising symbol
 *   Needs 2*Cq_r <= 32 in every row.  A typical key table costs 3 to 7 bytes.
 * Length kinds of cg_decode_job.lengths: CG_LENGTHS_I32 (the reference's int32) or CG_LENGTHS_U16. */
#define CG_TABLES_CDF 0
#define CG_TABLES_COUNTS 1
#define CG_TABLES_SPARSE 2
#define CG_LENGTHS_I32 0
#define CG_LENGTHS_U16 1

/* argument errors (returned) */
#define CG_OK 0
#define CG_E_NULL (-1)        /* a required pointer is NULL */
#define CG_E_SHAPE (-2)       /* non-positive or inconsistent extent */
#define CG_E_TOKENS (-3)      /* more than CG_MAX_TOKENS_PER_STREAM tokens in a coder call */
#define CG_E_LP (-4)          /* CDF length outside [2, CG_MAX_LP] / max_bins outside [1, 63] */
#define CG_E_ALIGN (-5)       /* pointer or stride breaks an alignment rule of the call */
#define CG_E_CAPACITY (-6)    /* scratch / workspace too small, or too many jobs */
#define CG_E_DTYPE (-7)       /* unknown 16-bit float code */
#define CG_E_CUDA (-8)        /* the CUDA runtime refused the launch; see cg_last_cuda_error */
#define CG_E_HIST (-9)        /* ntokens >= 65536: the reference's uint16 histogram would wrap */

/* device-reported conditions (bits OR-ed into *status) */
#define CG_S_STREAM_OVERFLOW 1 /* an encoded stream needed more bytes than its scratch row */
#define CG_S_BAD_LENGTHS 2     /* negative length, or lengths reach past the byte array */
#define CG_S_BAD_SYMBOL 4      /* a symbol outside [0, Lp-2] was met while encoding */
#define CG_S_COUNT_OVERFLOW 8  /* a histogram count above 255: the byte-count tables are not usable */
#define CG_S_BAD_TABLE 16     /* CG_TABLES_SPARSE offsets reach past the table set (read as zero counts) */

/*
 * Sizes in bytes of the buffers a caller allocates for the fused calls, for one chunk of
 * `ntokens` tokens with `nrows` = 2L rows of `nchannels` channels (no counterpart in the reference,
 * whose torch ops allocate as they go).  Returns CG_E_SHAPE for non-positive extents.
 */
typedef struct cg_workspace_sizes {
    int64_t nsub;              /* sub-chunks of the chunk: ceil(ntokens / 256) */
    int64_t scratch_stride;    /* bytes per stream in the encoder's scratch: CG_STREAM_CAPACITY, rounded to 4 */
    int64_t encode_scratch;    /* cg_encode_chunk scratch:        nsub * nrows * nchannels * scratch_stride */
    int64_t encode_lengths;    /* cg_encode_chunk lengths_out:    nsub * nrows * nchannels * 4 */
    int64_t encode_group_off;  /* cg_encode_chunk group_off_out:  nsub * nrows * ceil(nchannels/128) * 8 */
    int64_t encode_sub_off;    /* cg_encode_chunk sub_off_out:    (nsub + 1) * 8 */
    int64_t decode_group_off;  /* cg_decode_offsets group_off_out, per job (= per sub-chunk):
                                  nrows * ceil(nchannels/128) * 8 */
    int64_t symbols;           /* cg_quantize_cdf sym_out:        nrows * ntokens * nchannels */
} cg_workspace_sizes;
int cg_workspace_bytes(int nrows, int ntokens, int nchannels, cg_workspace_sizes *out_host);

const char *cg_version(void);
const char *cg_status_string(int code);
/* text of the last CUDA runtime error seen by this library on the calling thread */
const char *cg_last_cuda_error(void);

/* ------------------------------------------------------------------------------------------
 * torchac_cuda entry points
 * ------------------------------------------------------------------------------------------ */

/*
 * Replaces torchac_cuda.calculate_cdf (cal_cdf.cu:68-129, kernel cal_cdf.cu:17-59).
 * sym: int8 [nrows, ntokens, nchannels] with element strides sym_strides[3];
 * cdf_out: int16 [nrows, nchannels, max_bins + 1], contiguous.
 * cdf[i] = (uint16)((0xFFFF - max_bins) * #{sym < i} / ntokens) + i.  max_bins < 64 as in
 * cal_cdf.cu:73; ntokens < 65536 (the reference's uint16 counters wrap there).
 */
int cg_calculate_cdf(const int8_t *sym, const int64_t sym_strides[3], int nrows, int ntokens,
                     int nchannels, int max_bins, int16_t *cdf_out, void *stream);

/*
 * Replaces torchac_cuda.encode_fast_new (torchac_kernel_enc_new.cu:355-451, kernel :222-325).
 * cdf: int16 [nrows, nchannels, lp]; sym: int8 [nrows, ntokens, nchannels] (strided);
 * out_buf: uint8 [nrows, nchannels, out_stride], out_stride a multiple of 4 and out_buf 4-byte
 * aligned; out_lengths: int32 [nrows, nchannels].  Bytes of a row past the stream's length are
 * left as they were (the reference zero-fills nothing either).  A stream that needs more than
 * out_stride bytes is truncated, its full length is still reported and CG_S_STREAM_OVERFLOW is
 * raised (the reference overruns its 256-byte shared-memory row silently).
 */
int cg_encode_padded(const int16_t *cdf, const int8_t *sym, const int64_t sym_strides[3],
                     int nrows, int ntokens, int nchannels, int lp, uint8_t *out_buf,
                     int64_t out_stride, int32_t *out_lengths, int32_t *status, void *stream);

/*
 * Replaces torchac_cuda.decode_fast_new (torchac_kernel_dec_new.cu:314-393, kernel :75-186).
 * streams: uint8 [nrows, nchannels, stream_stride]; lengths: int32 [nrows, nchannels];
 * out: uint8 symbols [nrows, ntokens, nchannels] with element strides out_strides[3].
 * Reads past a stream's length see zero bits (torchac_kernel_dec_new.cu:229-232).
 */
int cg_decode_padded(const int16_t *cdf, const uint8_t *streams, int64_t stream_stride,
                     const int32_t *lengths, uint8_t *out, const int64_t out_strides[3],
                     int nrows, int ntokens, int nchannels, int lp, int32_t *status, void *stream);

/*
 * Replaces torchac_cuda.decode_fast_prefsum (torchac_kernel_dec_new.cu:403-479, kernel :189-304).
 * bytes: uint8 [nbytes], the streams back to back in (row, channel) order;
 * prefsum: int64 [nrows, nchannels], INCLUSIVE prefix sum of the stream lengths
 * (cachegen_decoder.py:70); stream g spans [prefsum[g-1], prefsum[g]), from 0 for g = 0.
 */
int cg_decode_prefsum(const int16_t *cdf, const uint8_t *bytes, int64_t nbytes,
                      const int64_t *prefsum, uint8_t *out, const int64_t out_strides[3],
                      int nrows, int ntokens, int nchannels, int lp, int32_t *status,
                      void *stream);

/*
 * The same decode as cg_decode_prefsum with one WARP per stream (lane m holds table entry m, a ballot
 * finds the symbol).  Same results; lp <= 33.  Kept as the measured alternative to the thread-per-stream
 * layout of every other decoder entry point: it is several times slower and nothing else uses it.
 */
int cg_decode_prefsum_warp(const int16_t *cdf, const uint8_t *bytes, int64_t nbytes,
                           const int64_t *prefsum, uint8_t *out, const int64_t out_strides[3],
                           int nrows, int ntokens, int nchannels, int lp, int32_t *status,
                           void *stream);

/* ------------------------------------------------------------------------------------------
 * fused encode side
 * ------------------------------------------------------------------------------------------ */

/*
 * Replaces _split_kv + torch_quant_vectorized (x2) + torch.cat + calculate_cdf (x2) + torch.cat
 * of encode_function (cachegen_encoder.py:72-83,42-59,257-267) in two launches.
 *
 * kv: 16-bit floats, element (layer l, k/v j, token t, head h, d) at
 *     kv[l*s_layer + j*s_kv + t*s_token + h*s_head + d]  (innermost stride 1).
 *     "vllm" blob [L,2,T,H,D]: s_layer=2*T*H*D, s_kv=T*H*D, s_token=H*D, s_head=D.
 *     "huggingface" blob [L,2,H,T,D]: s_layer=2*H*T*D, s_kv=H*T*D, s_token=D, s_head=T*D.
 * bins: float32 [2*L] on the device, key bins then value bins (make_key_bins / make_value_bins,
 *     cachegen_encoder.py:311-322).
 * sym_out: int8 [2L, T, C] contiguous, C = H*D;  scales_out: 16-bit [2L, T] (max_tensors_key
 *     then max_tensors_value, same dtype as kv);  cdf_out: int16 [2L, C, max_bins+1].
 * The reference builds key and value tables with their own max_bins and concatenates them,
 * which only works when both are equal (cachegen_encoder.py:265-267); pass that one value.
 * counts_out (may be NULL): the CG_TABLES_COUNTS form of the same tables, with table_row_off [2L]
 *     as described there; CG_S_COUNT_OVERFLOW is raised in *status when a count does not fit a byte.
 */
int cg_quantize_cdf(const void *kv, int dtype, int64_t s_layer, int64_t s_kv, int64_t s_token,
                    int64_t s_head, int nlayers, int ntokens, int nheads, int head_size,
                    const float *bins, int max_bins, int8_t *sym_out, void *scales_out,
                    int16_t *cdf_out, uint8_t *counts_out, const int64_t *table_row_off,
                    int32_t *status, void *stream);

/*
 * The two halves of cg_quantize_cdf on their own, for encoding one chunk at several bin settings
 * (the quality levels of cachegen_basics.py:33-68, which src/utils.py:294-314 chooses among per chunk):
 * the scales do not depend on the bins, so cg_row_absmax runs once and cg_quantize_cdf_scaled once per
 * level with `scales` as an input.  Arguments as for cg_quantize_cdf.
 */
int cg_row_absmax(const void *kv, int dtype, int64_t s_layer, int64_t s_kv, int64_t s_token,
                  int64_t s_head, int nlayers, int ntokens, int nheads, int head_size,
                  void *scales_out, void *stream);
int cg_quantize_cdf_scaled(const void *kv, int dtype, int64_t s_layer, int64_t s_kv, int64_t s_token,
                           int64_t s_head, int nlayers, int ntokens, int nheads, int head_size,
                           const float *bins, int max_bins, const void *scales, int8_t *sym_out,
                           int16_t *cdf_out, uint8_t *counts_out, const int64_t *table_row_off,
                           int32_t *status, void *stream);

/*
 * cg_quantize_cdf with anchor-token delta coding.  No counterpart in the reference, whose serializer
 * quantises every token on its own (cachegen_encoder.py:42-59); delta_group == 0 is exactly
 * cg_quantize_cdf.  With delta_group = G (a power of two, 2..256): in every row r with
 * res_bins[r] > 0 (float32 [2*L] on the device, 1 <= res_bins[r] // 2 - 1 <= bins[r] // 2 - 1), token t
 * of the call with t % G != 0 is coded as its difference from the DEQUANTISED first token a of its
 * group, as a decoder reconstructs it:
 *     x^a = cast(((sym_a - Cq_a) / Cq_a) * max_a)       r = cast(float(x_t) - float(x^a))
 *     max_t = amax|r|    sym_t = round(float(r) * (Cq_r / max_t) + Cq_r) + (Cq_a - Cq_r)
 * (casts to the KV dtype; Cq_a = bins[r] // 2 - 1, Cq_r = res_bins[r] // 2 - 1).  scales_out holds
 * max_t of the residual for those tokens; symbols of both kinds centre on Cq_a and share the row's
 * tables.  Other rows and the first token of every group are quantised as cg_quantize_cdf does.
 * The decoder must be given the same delta_group and res_bins (cg_decode_dequant_delta).  Three launches.
 */
int cg_quantize_cdf_delta(const void *kv, int dtype, int64_t s_layer, int64_t s_kv, int64_t s_token,
                          int64_t s_head, int nlayers, int ntokens, int nheads, int head_size,
                          const float *bins, int max_bins, int delta_group, const float *res_bins,
                          int8_t *sym_out, void *scales_out, int16_t *cdf_out, uint8_t *counts_out,
                          const int64_t *table_row_off, int32_t *status, void *stream);

/*
 * Byte counts (CG_TABLES_COUNTS, as cg_quantize_cdf writes them) -> CG_TABLES_SPARSE parts.  No
 * counterpart in the reference.  counts / count_row_off [nrows]: the dense counts and their row
 * offsets; bins: float32 [nrows] on the device.  group_off_out: uint32 [nrows * ceil(nchannels/128) + 1];
 * masks_out with mask_row_off [nrows] (device; row r's masks start mask_row_off[r] bytes in, 4-byte
 * aligned; 2 bytes per channel for rows with 2*Cq <= 16, else 4); counts_out: room for every count
 * (the size of the dense counts is always enough); group_off_out's last entry tells how many were
 * written.  The caller makes sure that no row has 2*Cq > 32.  Three launches.
 */
int cg_pack_sparse_tables(const uint8_t *counts, const int64_t *count_row_off, const float *bins,
                          int nrows, int nchannels, uint32_t *group_off_out, void *masks_out,
                          const int64_t *mask_row_off, uint8_t *counts_out, void *stream);

/*
 * Replaces the sub-chunk loop of encode_function: encode_fast_new + the length bookkeeping of
 * collect_bytes for every sub-chunk of a chunk (cachegen_encoder.py:269-292,210-242).
 * sym: int8 [nrows, ntokens, nchannels] contiguous, ntokens any positive number; the chunk is cut
 * in nsub = ceil(ntokens / 256) sub-chunks, all coded with the one table set `cdf`.
 * scratch: uint8 [nsub, nrows*nchannels, scratch_stride]  (scratch_stride % 4 == 0;
 *     CG_STREAM_CAPACITY(256) can never overflow);
 * lengths_out: int32 [nsub, nrows, nchannels];
 * group_off_out: int64 [nsub, ngroups], ngroups = nrows * ceil(nchannels / 128): exclusive byte
 *     offset, within its own sub-chunk, of the first stream of every 128-channel group;
 * sub_off_out: int64 [nsub + 1]: byte offset of every sub-chunk in the concatenation of all
 *     sub-chunks; the last entry is the total payload size.
 */
int cg_encode_chunk(const int16_t *cdf, const int8_t *sym, int nrows, int ntokens, int nchannels,
                    int lp, uint8_t *scratch, int64_t scratch_stride, int32_t *lengths_out,
                    int64_t *group_off_out, int64_t *sub_off_out, int32_t *status, void *stream);

/*
 * Second half of collect_bytes (cachegen_encoder.py:210-222): gathers the first `length` bytes of
 * every scratch row into bytes_out (uint8, sub_off[nsub] bytes, as sized by the caller after
 * reading sub_off_out of cg_encode_chunk), streams back to back in (sub-chunk, row, channel) order.
 * lengths, group_off and sub_off are the arrays cg_encode_chunk wrote.
 */
int cg_compact_streams(const uint8_t *scratch, int64_t scratch_stride, const int32_t *lengths,
                       const int64_t *group_off, const int64_t *sub_off, int nsub, int nrows,
                       int nchannels, uint8_t *bytes_out, void *stream);

/* ------------------------------------------------------------------------------------------
 * fused decode side
 * ------------------------------------------------------------------------------------------ */

/* One sub-chunk (CacheGenGPUBytestream, cachegen_basics.py:124-131) of one encoded chunk. */
typedef struct cg_decode_job {
    const void *tables;      /* table set of the chunk, see table_kind */
    const uint8_t *bytes;    /* the sub-chunk's streams, back to back */
    const void *lengths;     /* [nrows, nchannels] stream lengths (bytestream_lengths), see length_kind */
    const int64_t *group_off;/* [nrows*ceil(nchannels/128)] exclusive byte offset of each
                                128-channel group inside `bytes`: written by cg_decode_offsets */
    const void *scales_k;    /* 16-bit [nlayers, scale_stride]: max_tensors_key, at this
                                sub-chunk's first token */
    const void *scales_v;    /* 16-bit [nlayers, scale_stride]: max_tensors_value, likewise */
    void *out;               /* 16-bit KV, element (layer 0, key, this sub-chunk's first token,
                                head 0, d 0) of the output blob */
    const int64_t *table_row_off; /* CG_TABLES_COUNTS: [nrows] row offsets into `tables`;
                                CG_TABLES_SPARSE: [nrows + 1] row offsets into its masks */
    int64_t nbytes;          /* size of `bytes` */
    int64_t tables_nbytes;   /* CG_TABLES_COUNTS and CG_TABLES_SPARSE: size of `tables` in bytes; reads
                                are kept inside it (CG_S_BAD_TABLE otherwise) */
    int32_t ntokens;         /* tokens in this sub-chunk, 1..256 */
    int32_t scale_stride;    /* elements between consecutive layers in scales_k / scales_v
                                (= the chunk's token count, over which its tables were built) */
    int32_t table_kind;      /* CG_TABLES_CDF, CG_TABLES_COUNTS or CG_TABLES_SPARSE */
    int32_t length_kind;     /* CG_LENGTHS_I32 or CG_LENGTHS_U16 */
} cg_decode_job;

/*
 * Exclusive offsets of every 128-channel group of every job (the cumsum of
 * cachegen_decoder.py:70, computed per group instead of per stream).  Writes
 * group_off_out[j * ngroups + g] for the njobs jobs; fill cg_decode_job.group_off with
 * group_off_out + j * ngroups.  Only jobs[].lengths and jobs[].nbytes are read.
 * Raises CG_S_BAD_LENGTHS when a job's lengths are negative or do not sum to its nbytes.
 */
int cg_decode_offsets(const cg_decode_job *jobs_host, int njobs, int nrows, int nchannels,
                      int64_t *group_off_out, int32_t *status, void *stream);

/*
 * Replaces decode_function_gpu + do_dequantize (x2) + torch.stack + reshape + permute + cast of
 * CacheGenDeserializer.from_bytes (cachegen_decoder.py:78-112,24-34,159-173) in one launch:
 * arithmetic decode, (sym - Cq) / Cq * max in fp32, one round-to-nearest cast, store into the
 * final KV blob.
 * Output element (layer l, k/v j, token t, head h, d) of a job is written at
 *     job.out[l*o_layer + j*o_kv + t*o_token + h*o_head + d]
 * (strides as for cg_quantize_cdf; "vllm" gives [L,2,T,H,D], "huggingface" [L,2,H,T,D]).
 * bins: float32 [2*nlayers] on the device (key bins then value bins, cachegen_decoder.py:122-135);
 * scale_dtype: type of scales_k / scales_v; out_dtype: type of the output
 * (the reference returns bf16 for "vllm" and fp16 for "huggingface", cachegen_decoder.py:169-173).
 * njobs <= CG_MAX_DECODE_JOBS; all jobs share nlayers, nheads, head_size, lp and the strides.
 */
int cg_decode_dequant(const cg_decode_job *jobs_host, int njobs, int nlayers, int nheads,
                      int head_size, int lp, const float *bins, int scale_dtype, int out_dtype,
                      int64_t o_layer, int64_t o_kv, int64_t o_token, int64_t o_head,
                      int32_t *status, void *stream);

/*
 * cg_decode_dequant for chunks written by cg_quantize_cdf_delta (no counterpart in the reference;
 * delta_group == 0 is exactly cg_decode_dequant).  In rows with res_bins[r] > 0 a token that is not the
 * first of its group of delta_group decodes to
 *     cast_out(float(cast_kv(v_anchor)) + ((sym - Cq_a) / Cq_r) * max_t)
 * where v_anchor is the fp32 value of the group's first token and cast_kv rounds to scale_dtype, the
 * KV dtype the encoder saw.  Every job must start on a group boundary (sub-chunks of 256 tokens do).
 * Needs the layout of the two-channels-per-thread kernel: even head_size and strides, 4-byte aligned
 * output (CG_E_ALIGN otherwise).
 */
int cg_decode_dequant_delta(const cg_decode_job *jobs_host, int njobs, int nlayers, int nheads,
                            int head_size, int lp, const float *bins, int delta_group,
                            const float *res_bins, int scale_dtype, int out_dtype, int64_t o_layer,
                            int64_t o_kv, int64_t o_token, int64_t o_head, int32_t *status, void *stream);

/*
 * No counterpart in the reference.  The same work as cg_decode_offsets followed by cg_decode_dequant,
 * for callers that cannot provide the group-offset workspace because they cannot allocate device
 * memory where the decode runs: a serving engine that has already handed every free byte of HBM to
 * its KV block pool, or a latency-critical worker that must keep cudaMalloc (which synchronises the
 * whole device) off its path.  The offsets live in an array built into the library instead
 * (CG_STATIC_OFFSET_ENTRIES int64 values, 1 MiB, resident on every GPU that loads the library until
 * the process exits).
 *
 * jobs_host[].group_off is ignored.  Limit: njobs * 2*nlayers * ceil(nheads*head_size / 128) must not
 * exceed CG_STATIC_OFFSET_ENTRIES, otherwise CG_E_CAPACITY is returned and nothing is launched.
 * The call allocates nothing.  The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current) and remembers it; make that first call outside
 * any stream capture.  All calls on a device share the one array and it keeps the previous call's
 * contents: every entry a call reads it has written first, so nothing needs clearing, but two calls
 * whose kernels may overlap on the GPU (different streams, no ordering between them) race on it.
 */
#define CG_STATIC_OFFSET_ENTRIES 131072
int cg_decode_dequant_static(const cg_decode_job *jobs_host, int njobs, int nlayers, int nheads,
                             int head_size, int lp, const float *bins, int scale_dtype, int out_dtype,
                             int64_t o_layer, int64_t o_kv, int64_t o_token, int64_t o_head,
                             int32_t *status, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* CACHEGEN_B200_H */
