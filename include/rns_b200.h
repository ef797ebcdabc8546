/*
 * rns_b200.h - C ABI of the B200 (sm_100a) RNS linear library, librns_b200.so.
 *
 * Every entry point takes plain pointers and sizes, enqueues its work on the
 * stream it is given and returns a status code at once; none of them
 * allocates, frees or synchronises (the one set-up exception is documented at
 * its declaration).  Pointers named "d_*" are device pointers on the current
 * device; "moduli" is always a host array.  All matrices are row-major.
 *
 * Vocabulary: a *channel* is one modulus m_c of the residue number system; a
 * *plane* is the int8 matrix of centred residues of one channel; P is the
 * product of the active moduli.
 *
 * Each declaration cites the interface of the reference implementation
 * (Nek1tt/rns-llm v0.5) that it stands in for, as path:line inside that
 * project.
 */
#ifndef RNS_B200_H_
#define RNS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define RNS_API
#else
#define RNS_API __attribute__((visibility("default")))
#endif

/* Opaque stand-in for cudaStream_t so that C callers need no CUDA headers. */
typedef void* rns_stream_t;

#define RNS_MAX_CHANNELS 10   /* reference: csrc/rns_cuda.cu:963-975 accepts 2..10 */
#define RNS_TC_MAX_CHANNELS 8 /* channel count the tcgen05 kernel is instantiated for */
#define RNS_MAX_PEERS 7       /* other ranks of one NVLink domain that a launch can store to */

typedef enum rns_status {
    RNS_OK = 0,
    RNS_ERR_INVALID_ARGUMENT = 1, /* bad pointer, size, stride, enum value         */
    RNS_ERR_BAD_MODULI = 2,       /* not in [2,255] or not pairwise coprime        */
    RNS_ERR_UNSUPPORTED = 3,      /* valid request outside what the kernels cover  */
    RNS_ERR_OVERFLOW = 4,         /* P or a dot-product bound exceeds its type     */
    RNS_ERR_CUDA = 5,             /* a CUDA runtime/driver call failed             */
    RNS_ERR_DEVICE_TIMEOUT = 6    /* a bounded device-side wait expired            */
} rns_status;

/* Element type of the source integers handed to the encoders. */
typedef enum rns_int_type { RNS_INT8 = 0, RNS_INT16 = 1, RNS_INT32 = 2 } rns_int_type;

/* What the fused GEMM epilogue stores. */
typedef enum rns_out_type {
    RNS_OUT_INT64 = 0, /* exact integer, as the reference's workspace.output     */
    RNS_OUT_INT32 = 1, /* exact integer; requires P/2 < 2^31                     */
    RNS_OUT_F16 = 2,   /* dequantised: f16( f32(x)*row_scale*col_scale + bias )  */
    RNS_OUT_BF16 = 3,
    RNS_OUT_F32 = 4
} rns_out_type;

/* Floating type of an activation tensor given to the quantiser. */
typedef enum rns_float_type { RNS_F16 = 0, RNS_BF16 = 1, RNS_F32 = 2 } rns_float_type;

/* Text of the last error raised on the calling thread ("" if none). */
RNS_API const char* rns_last_error(void);

/* Library/ABI version: major*10000 + minor*100 + patch. */
RNS_API int rns_version(void);

/* ------------------------------------------------------------------------
 * Host-side constants
 * --------------------------------------------------------------------- */

/*
 * Validates moduli (each in [2,255], pairwise coprime: reference
 * src/rns_llm/reference.py:11-23) and writes the constants the reference keeps
 * per (device, moduli) in _DeviceConstants (backends/cuda_backend.py:48-66,
 * 137-166): reciprocals floor(2^32/m) [channels], pairwise inverses
 * inv[j*channels+i] = m_j^-1 mod m_i for j<i [channels*channels], and P.
 * Any output pointer may be NULL.  RNS_ERR_OVERFLOW when P > INT64_MAX.
 */
RNS_API int rns_host_constants(const int32_t* moduli, int channels,
                               int64_t* reciprocals, int32_t* pairwise_inverses,
                               int64_t* modulus_product);

/*
 * Smallest prefix length c >= min_channels with 2*bound < m_0*...*m_{c-1}
 * (reference src/rns_llm/adaptive.py:15-41).  Returns c, or a negative
 * rns_status: -RNS_ERR_OVERFLOW when even the full set is too small.
 */
RNS_API int rns_minimal_prefix_channels(const int32_t* moduli, int channels,
                                        int64_t absolute_bound, int min_channels);

/*
 * Host evaluation of the exact expressions the device epilogue and the
 * in-kernel encoder use (same source, compiled for the CPU).  For tests and
 * for callers that want to check a modulus set without a GPU; no counterpart
 * in the reference, whose device arithmetic cannot run on the host.
 *   rns_host_reconstruct: sums int32 [channels, count] (per-channel dot
 *     products, any representative) -> signed value, as csrc/rns_cuda.cu:
 *     442-476 would produce from the same accumulators, using the first
 *     `active` channels.
 *   rns_host_encode_centered_i8: int8 [count] -> centred planes int8
 *     [channels, count] through the packed single-fold encoder (count % 4 == 0,
 *     every modulus >= 86).
 */
RNS_API int rns_host_reconstruct(const int32_t* sums, int64_t count, const int32_t* moduli,
                                 int channels, int active, int64_t* out);
RNS_API int rns_host_encode_centered_i8(const int8_t* values, int64_t count,
                                        const int32_t* moduli, int channels, int8_t* out);
/*   rns_host_encode_reduced_i8: the fused kernel's default in-kernel encoder:
 *     one-step reduced residues (x - m for x >= 64, x + m for x < -64, moduli
 *     above 191 pass through): congruent to x, inside int8, any moduli. */
RNS_API int rns_host_encode_reduced_i8(const int8_t* values, int64_t count,
                                       const int32_t* moduli, int channels, int8_t* out);

/* ------------------------------------------------------------------------
 * Plane-level entry points: the six functions of the reference's FFI module
 * rns_llm._C (csrc/bindings.cpp:45-75), with raw pointers in place of tensors.
 * --------------------------------------------------------------------- */

/*
 * encode_int8 (csrc/bindings.cpp:46-49; kernel csrc/rns_cuda.cu:126-148):
 * canonical residues in [0, m).  d_out is uint8 [channels, elements].
 */
RNS_API int rns_encode_canonical_i8(const int8_t* d_values, int64_t elements,
                                    const int32_t* moduli, int channels,
                                    uint8_t* d_out, rns_stream_t stream);

/*
 * encode_centered (csrc/bindings.cpp:51-54; kernel csrc/rns_cuda.cu:98-124):
 * centred residues; C remainder then fold into [-floor(m/2), floor(m/2)], so
 * for an even modulus -m/2 stays negative.  d_out is int8 [channels, elements].
 */
RNS_API int rns_encode_centered(const void* d_values, rns_int_type type, int64_t elements,
                                const int32_t* moduli, int channels,
                                int8_t* d_out, rns_stream_t stream);

/*
 * matmul_residues (csrc/bindings.cpp:56-59; csrc/rns_cuda.cu:628-709):
 * canonical uint8 planes a [channels,M,K] x b [channels,K,N] -> canonical
 * uint8 [channels,M,N].  The reference's kernel_id (0..2) selects between
 * kernels with identical results; it is validated and otherwise ignored.
 */
RNS_API int rns_matmul_canonical_planes(const uint8_t* d_a, const uint8_t* d_b,
                                        const int32_t* moduli, int channels,
                                        int m, int k, int n, int kernel_id,
                                        uint8_t* d_out, rns_stream_t stream);

/*
 * matmul_centered_residues (csrc/bindings.cpp:61-64; csrc/rns_cuda.cu:711-816):
 * centred int8 planes -> centred int8 planes [channels,M,N].  kernel_id 0..3
 * (scalar, dp4a, dp4a_safe, cublas) is validated; every value runs the same
 * exact kernel.  kernel_id 3 keeps the reference's K%4==0 && N%4==0 check.
 */
RNS_API int rns_matmul_centered_planes(const int8_t* d_a, const int8_t* d_b,
                                       const int32_t* moduli, int channels,
                                       int m, int k, int n, int kernel_id,
                                       int8_t* d_out, rns_stream_t stream);

/*
 * decode_garner (csrc/bindings.cpp:66-69; csrc/rns_cuda.cu:416-440, 818-885):
 * centred int8 planes [channels, elements] -> signed int64 in (-P/2, P/2].
 */
RNS_API int rns_decode_garner(const int8_t* d_residues, int64_t elements,
                              const int32_t* moduli, int channels,
                              int64_t* d_out, rns_stream_t stream);

/*
 * matmul_centered_fused_out (csrc/bindings.cpp:71-74; csrc/rns_cuda.cu:887-980):
 * centred planes a [channels,M,K], b [channels,K,N] -> d_out int64 [M,N].
 * d_accumulators (int32 [channels,M,N]) is the caller's workspace as in the
 * reference and receives the raw per-channel sums.  lut_channels (0..2) is
 * validated and otherwise ignored: reduction happens in registers.  Keeps the
 * reference's K%4==0 && N%4==0 && 2<=channels<=10 checks.
 */
RNS_API int rns_matmul_centered_fused_out(const int8_t* d_a, const int8_t* d_b,
                                          const int32_t* moduli, int channels,
                                          int m, int k, int n, int lut_channels,
                                          int32_t* d_accumulators, int64_t* d_out,
                                          rns_stream_t stream);

/* ------------------------------------------------------------------------
 * The fused sm_100a path
 * --------------------------------------------------------------------- */

/*
 * Arguments of rns_linear_fused.  Replaces, in one launch, the chain
 * encode_centered(a) -> cublasGemmStridedBatchedEx -> fused_reduce_garner_kernel
 * -> eager dequantisation of the reference (backends/cuda_backend.py:514-539,
 * 398-459; csrc/rns_cuda.cu:478-523, 442-476; layers/rns_linear.py:264, 272-275).
 *
 * Activations come either as source integers d_a int8 [M,K] (row stride lda,
 * residues formed inside the kernel) or as planes d_a_planes int8
 * [channels,M,K] produced by rns_quantize_activations / rns_encode_centered
 * (row stride lda, plane stride a_plane_stride); exactly one is non-NULL.
 * Weights are ALWAYS source integers d_w int8 [N,K] (the nn.Linear layout, row
 * stride ldw): one byte per value whatever the channel count; their residues
 * are formed inside the kernel.
 *
 * Packed tile layouts.  TMA moves a [rows x 64 B] box of a row-major matrix as
 * one request per 64-byte row, which bounds the load rate far below what the
 * tensor cores consume.  The packed layouts store every 64-byte-deep tile row
 * block contiguously and already in the shared-memory (64-byte swizzled) image,
 * so that one bulk copy fills a pipeline stage:
 *   weights      [K_pad/64][N_pad][64]        N_pad = N rounded up to 384,
 *   activations  [M_pad/128][K_pad/64][128][64]             (source integers)
 *   planes       [M_pad/128][K_pad/64][channels][128][64]   M_pad = M up to 256,
 * K_pad = K rounded up to 64 (the weight side is zero there).  Inside a 64-byte
 * row the 16-byte chunk j of row r is stored at chunk j ^ ((r >> 1) & 3).
 * rns_pack_weight / rns_quantize_activations / rns_encode_planes_packed write
 * these layouts; lda, ldw and a_plane_stride are ignored for packed operands.
 *
 * d_active_channels, when non-NULL, points to a device int c (2..channels):
 * only the first c moduli are used (adaptive prefix, backends/cuda_backend.py:
 * 573-622, decided on the device by rns_select_channels).  Honoured by the
 * general kernel and, with tiled planes (a_tile_rows), by variant 4 for 4 or 5
 * channels without w_channel_stride and output copies.
 *
 * Integer output types store x = sum_k a[m,k]*w[n,k] reconstructed and
 * recentred exactly as csrc/rns_cuda.cu:380-414.  Floating output types store
 * type( f32(x) * row_scale[m*row_scale_stride] * col_scale[n] (+ bias[n]) )
 * with every product and the sum rounded to f32 in that order, which is the
 * arithmetic of layers/rns_linear.py:272-275; row_scale_stride is 0 for a
 * per-tensor activation scale and 1 for per-row scales.
 *
 * d_status, when non-NULL, is a device int the kernel sets to a non-zero
 * rns_status (RNS_ERR_DEVICE_TIMEOUT) if a bounded wait expires.
 *
 * Requirements of the tensor-core kernel: K % 16 == 0, lda/ldw/a_plane_stride
 * multiples of 16, 16-byte aligned bases, 2 <= channels <= 8 (and every modulus
 * >= 86 when exact_residues is set).  Anything else
 * returns RNS_ERR_UNSUPPORTED; callers then use the plane-level functions.
 * K * 128 * 128 must not exceed INT32_MAX (K <= 131071): the per-channel sums
 * are int32, as the reference's cuBLAS accumulators are (backends/
 * cuda_backend.py:240); a larger K returns RNS_ERR_OVERFLOW.
 */
typedef struct rns_linear_args {
    int32_t m, n, k;
    int32_t channels;
    int32_t moduli[RNS_MAX_CHANNELS];
    const int8_t* d_a;
    const int8_t* d_a_planes;
    int64_t lda;
    int64_t a_plane_stride;
    const int8_t* d_w;
    int64_t ldw;
    const int32_t* d_active_channels;
    void* d_out;
    int64_t ldo;              /* in elements of the output type */
    int32_t out_type;         /* rns_out_type */
    const float* d_row_scale; /* floating outputs only */
    int32_t row_scale_stride; /* 0 or 1 */
    const float* d_col_scale; /* [N], floating outputs only */
    const float* d_bias;      /* [N] or NULL */
    int32_t* d_status;
    int32_t tile_n;           /* 0 = choose; else 16..128, multiple of 16 */
    int32_t tile_k;           /* 0 = choose; else 64 or 128 (128: plain layouts only) */
    int32_t a_packed;         /* 1: d_a / d_a_planes is in the packed tile layout */
    int32_t w_packed;         /* 1: d_w is in the packed tile layout (rns_pack_weight) */
    int32_t pair_mode;        /* 1: two-CTA tiles (256 x tile_n), 0: one CTA per tile, 2: choose */
    int32_t enc_groups;       /* 0 = choose; else 1, 2 or 4 groups of encoder warps */
    int32_t enc_stages;       /* 0 = choose; else depth of the operand ring (1..8) */
    int32_t sub_blocks;       /* 0 = choose; else K blocks of tile_k bytes per pipeline stage (1..4) */
    int32_t variant;          /* 0 = choose; 1: operands staged in shared memory; 2: weights as
                                 tensor-memory operands (packed planes + packed weights, 2..5
                                 channels; tile_n then means tokens per tile: 32, 64 or 128);
                                 3 and 4: two-CTA feature-major kernels (see a_tile_rows); 4, the
                                 one 0 resolves to for that layout, gives every residue channel
                                 the int8 weight itself as its weight operand (a representative
                                 of the same residue class: the sums differ by multiples of the
                                 modulus, the reconstructed integers not at all), 3 encodes the
                                 canonical weight residues per channel inside the kernel */
    int32_t exact_residues;   /* 1: in-kernel residues exactly centred (|r| <= m/2; needs every
                                 modulus >= 86); 0: one-step reduced residues (any moduli) */
    int32_t a_tile_rows;      /* packed planes only: token rows per packed tile. 0 or 128: the layout
                                 above.  64 (up to four channels), 48 (five) or 32 (six): tiles of that many
                                 rows, [M_pad/rows][K_pad/64][channels][rows][64], written by
                                 rns_quantize_activations_tiled; selects the two-CTA feature-major
                                 kernels (variants 3 and 4), which need 4 to 6 channels (variant 3: 4 or 5) and K >= 512 */
    uint32_t* d_absmax_out;   /* NULL, or device word that receives the bit pattern of
                                 max |y| over the floating outputs as stored (variants 3 and 4 only;
                                 two words: the launch clears both and uses [1] as a counter): the per-tensor absmax the NEXT
                                 layer's quantiser needs, so that it can skip its own pass over
                                 the activations (layers/rns_linear.py:239-240 of the reference) */
    int32_t n_out_copies;     /* variants 3 and 4, floating outputs: the tile is ALSO stored, at the same
                                 offsets (same ldo), into these buffers - the same output slot in
                                 the memory of the other ranks of a column-sharded layer, mapped
                                 into this process (peer memory over NVLink; plain stores only).
                                 The exchange then runs under the GEMM instead of in an all-gather
                                 after it; the ranks still have to meet (a barrier) before anyone
                                 reads.  With d_absmax_out, d_absmax_copies[g] receives the finished
                                 word too (d_absmax_out then needs two words: [1] counts CTAs). */
    void* d_out_copies[RNS_MAX_PEERS];
    uint32_t* d_absmax_copies[RNS_MAX_PEERS];
    int32_t* d_wait_info;     /* NULL, or device int32[4], zero before the launch: when a bounded
                                 wait expires the first CTA to give up writes {wait code =
                                 role << 20 | pipeline stage, blockIdx.x, blockIdx.y, kernel form}
                                 here, so that the host can say where the kernel stopped */
    int64_t w_channel_stride; /* 0: d_w is ONE quantised int8 matrix, the source of every channel's weight
                                 operand.  Else (variant 0 / 4, tiled planes, 4..6 channels): d_w holds
                                 `channels` packed int8 matrices this many bytes apart (a multiple of 16;
                                 at least rns_packed_weight_bytes(n, k)), matrix c = the centred residues
                                 mod moduli[c] of a weight whose source integers are wider than int8
                                 (quant_bits 12 / 16 of layers/rns_linear.py:45-46, 96-98 of the reference;
                                 its backend caches the same planes, 4 bytes per value) */
    int32_t out_copies_multicast; /* 1: d_out_copies[0] and d_absmax_copies[0] (n_out_copies = 1) are NVLink
                                 multicast addresses (NVLS: one mapping that covers the same slot on every
                                 rank, this one included); the epilogue then issues ONE multimem.st per
                                 16 bytes instead of a store per peer, and the switch replicates it.  Needs
                                 two-byte outputs, N a multiple of 128, ldo a multiple of 8 and 16-byte
                                 aligned bases (only the row-wide store path has a multicast form) */
    int32_t groups;           /* 0: an ordinary call.  >= 1 (variant 0 / 4, tiled planes, one weight matrix, no
                                 prefix, no copies): that many independent m x k x n problems in one launch -
                                 the grouped multi-head QK^T / AV products the reference lists as open work
                                 (docs/OPTIMIZATIONS_V04.md:49; benchmarks/benchmark_attention.py:107-113
                                 times one head).  d_a_planes: the tiled planes of the [groups * m, k] matrix
                                 (m a multiple of 2 * a_tile_rows); d_w: the packed [groups * n, k] matrix
                                 (n a multiple of 8; problem g multiplies rows g * n .. g * n + n - 1);
                                 d_out: [groups][m][ldo]; scales and bias are shared by the problems.
                                 K may be as small as 64 here */
} rns_linear_args;

RNS_API int rns_linear_fused(const rns_linear_args* args, rns_stream_t stream);

/* Bytes of the packed layouts (see rns_linear_args). */
RNS_API int64_t rns_packed_weight_bytes(int n, int k);
RNS_API int64_t rns_packed_activation_bytes(int m, int k, int channels /* 1 = source integers */);
/* ... and of packed planes in tiles of tile_rows token rows (rns_linear_args.a_tile_rows);
 * M is padded to a multiple of 2 * tile_rows, the token tile of the two-CTA kernel. */
RNS_API int64_t rns_packed_planes_bytes(int m, int k, int channels, int tile_rows);
/* Token rows per packed tile that the two-CTA kernel wants for this channel count (64 up to
 * four channels, 48 for five, 32 for six), or 0 when it does
 * not cover it (then use the 128-row layout and variants 0..2). */
RNS_API int rns_pair_tile_rows(int channels, int k);

/*
 * Repacks quantised weights d_w int8 [N,K] (row stride ldw) into the packed
 * layout (zero padded), once per weight: the packed matrix replaces the plain
 * one, so a cached weight still costs one byte per value.  No reference
 * counterpart (the reference caches `channels` planes, backends/cuda_backend.py:
 * 464-487).  rns_unpack_weight is the inverse, for callers that ask for the
 * plain matrix or its planes again.
 */
RNS_API int rns_pack_weight(const int8_t* d_w, int n, int k, int64_t ldw, int8_t* d_packed,
                            rns_stream_t stream);
RNS_API int rns_unpack_weight(const int8_t* d_packed, int n, int k, int8_t* d_w, int64_t ldw,
                              rns_stream_t stream);

/*
 * Centred planes of already-quantised activations d_a int8 [M,K] (row stride
 * lda) in the packed planes layout: the activation encode of
 * backends/cuda_backend.py:532 for the large-M path.
 */
RNS_API int rns_encode_planes_packed(const int8_t* d_a, int m, int k, int64_t lda,
                                     const int32_t* moduli, int channels, int8_t* d_planes_packed,
                                     rns_stream_t stream);
/* The same in tiles of tile_rows token rows ([M_pad/rows][K_pad/64][channels][rows][64],
 * rns_linear_args.a_tile_rows; rns_packed_planes_bytes gives the size): the integer entry
 * of the two-CTA kernels. */
RNS_API int rns_encode_planes_tiled(const int8_t* d_a, int m, int k, int64_t lda,
                                    const int32_t* moduli, int channels, int tile_rows,
                                    int8_t* d_planes_packed, rns_stream_t stream);

/* 1 when rns_linear_fused accepts this problem, 0 when it would return
 * RNS_ERR_UNSUPPORTED (the role of CudaRNSBackend.cublas_compatible,
 * backends/cuda_backend.py:224-239). */
RNS_API int rns_linear_fused_supported(const int32_t* moduli, int channels, int k,
                                       int64_t lda, int64_t ldw);

/*
 * Activation quantiser: RNSLinear._symmetric_scale + _quantize
 * (layers/rns_linear.py:154-166, 239-241) and, optionally, the activation
 * encode of backends/cuda_backend.py:532, in at most two launches and without
 * a host round trip.
 *
 *   scale = max(absmax / quant_max, FLT_EPSILON)   (per tensor, or per row when
 *                                                   per_row != 0)
 *   q     = clamp(rint(x / scale), -quant_max, quant_max)      (ties to even)
 *
 * d_x is the logical [M,K] matrix.  Element (r,c) is read at
 *   d_x[(c / col_block) * col_block_stride + r * ldx + (c % col_block)]
 * (all in elements): col_block <= 0 means a plain matrix with row stride ldx;
 * col_block = K/G, col_block_stride = M*K/G, ldx = K/G reads the layout an
 * all-gather of G column shards [M,K/G] leaves behind, so the gathered output
 * of a column-sharded layer feeds the next layer without a transposing copy.
 * Outputs: d_q int8 [M,K]
 * (may be NULL when only planes are wanted), d_planes int8 [channels,M,K]
 * (NULL to skip) - both in the packed tile layouts of rns_linear_args when
 * packed_out != 0 (sizes: rns_packed_activation_bytes); the plain planes hold
 * centred residues as the reference's encode does, the packed planes, which only
 * feed the tensor cores, one-step reduced residues (congruent, |r| <= 64 for the
 * moduli just below 128; rns_host_encode_reduced_i8 states them) -,
 * d_scale float [1] or [M], d_row_l1_max int32 [1] = max_m
 * sum_k |q[m,k]| (NULL to skip; input of rns_select_channels).
 * d_scratch: 16 bytes of device scratch owned by the caller's stream (used
 * only by the two-launch per-tensor path, M*K > 32 Ki elements).
 * quant_max must be 127 (8-bit sources).
 */
RNS_API int rns_quantize_activations(const void* d_x, rns_float_type type,
                                     int m, int k, int64_t ldx,
                                     int col_block, int64_t col_block_stride,
                                     int per_row, int quant_max,
                                     const int32_t* moduli, int channels,
                                     int8_t* d_q, int8_t* d_planes, int packed_out,
                                     float* d_scale,
                                     int32_t* d_row_l1_max, void* d_scratch,
                                     rns_stream_t stream);

/*
 * The same quantiser with two extensions used by layer stacks (no reference
 * counterpart: the reference recomputes the absmax in eager torch for every layer):
 *   tile_rows          token rows per packed tile of d_planes (0/128 as above, or
 *                      rns_pair_tile_rows());
 *   d_absmax_parts     NULL, or `absmax_parts` device words `absmax_part_stride`
 *                      words apart, each the bit pattern of a non-negative float:
 *                      their maximum is taken as the tensor's absmax and the
 *                      quantiser's own pass over the activations is skipped (per-tensor
 *                      scale only).  A previous layer's d_absmax_out provides one word;
 *                      a column-sharded layer provides one word per rank.
 */
RNS_API int rns_quantize_activations_tiled(const void* d_x, rns_float_type type,
                                           int m, int k, int64_t ldx,
                                           int col_block, int64_t col_block_stride,
                                           int per_row, int quant_max,
                                           const int32_t* moduli, int channels,
                                           int8_t* d_q, int8_t* d_planes, int packed_out,
                                           int tile_rows, float* d_scale,
                                           int32_t* d_row_l1_max, void* d_scratch,
                                           const uint32_t* d_absmax_parts, int absmax_parts,
                                           int64_t absmax_part_stride, rns_stream_t stream);

/*
 * Row-L1 maximum of already-quantised activations: max_m sum_k |a[m,k]|, the
 * quantity select_adaptive_variant reads back with .item()
 * (backends/cuda_backend.py:591), left on the device instead.
 */
RNS_API int rns_row_l1_max_i8(const int8_t* d_a, int m, int k, int64_t lda,
                              int32_t* d_row_l1_max, rns_stream_t stream);

/*
 * On-device adaptive prefix selection (backends/cuda_backend.py:573-601 +
 * src/rns_llm/adaptive.py:15-52): bound = *d_row_l1_max * max_abs_weight;
 * *d_active_channels = smallest c >= min_channels with 2*bound < prod(m[:c]).
 * When even the full set is too small the reference raises OverflowError; here
 * *d_active_channels = channels and *d_status = RNS_ERR_OVERFLOW (if given).
 * d_meta, when non-NULL, receives int64 {channels, bound, capacity} for
 * last_adaptive_metadata, to be read lazily.  d_histogram, when non-NULL, is
 * int64 [RNS_MAX_CHANNELS+1]; entry [c] is incremented when c channels are
 * chosen (the adaptive_channels_{c} counters of backends/cuda_backend.py:599,
 * kept on the device and read only when statistics are asked for).
 */
RNS_API int rns_select_channels(const int32_t* d_row_l1_max, int32_t max_abs_weight,
                                const int32_t* moduli, int channels, int min_channels,
                                int32_t* d_active_channels, int64_t* d_meta,
                                int64_t* d_histogram, int32_t* d_status, rns_stream_t stream);

/*
 * Weight quantiser: per-output-channel symmetric int8 of layers/rns_linear.py:
 * 183-184 kept in the nn.Linear layout [N,K] (no transpose, no planes).
 * d_w is [N,K] (row stride ldw elements); d_wq int8 [N,K]; d_scale float [N];
 * d_max_abs int32 [1] = max |wq| (NULL to skip; feeds rns_select_channels).
 */
RNS_API int rns_quantize_weight(const void* d_w, rns_float_type type, int n, int k,
                                int64_t ldw, int quant_max, int8_t* d_wq, float* d_scale,
                                int32_t* d_max_abs, rns_stream_t stream);

/*
 * Few-token linear in ONE launch (decode steps, merged single-token requests): the
 * whole of RNSLinear.forward (layers/rns_linear.py:237-275: absmax, quantise, encode,
 * per-channel products, reconstruction, dequantise, bias) for M <= 32 tokens, where
 * the reference pays about 17 launches and this library's two-step path two.  Needs no
 * scratch memory at all.
 *   d_x      activations [M,K], row stride ldx: floating (x_type = rns_float_type;
 *            quantised per tensor, or per row when per_row != 0) or already-quantised
 *            int8 (x_type = -1; the merged activations of
 *            matmul_prepared_fused_requests, backends/cuda_backend.py:647-703)
 *   d_out    [M,N] of out_type: exact int64 / int32, or F16 / BF16 / F32 =
 *            type(f32(x) * s_a * col_scale[n] + bias[n]) (s_a = 1 for int8 activations)
 * rns_linear_small_supported: M <= 32, K % 16 == 0, 2..6 channels, channels * K <=
 * 196608; anything else returns RNS_ERR_UNSUPPORTED (use rns_linear_fused).
 */
RNS_API int rns_linear_small_supported(int m, int k, int channels);
RNS_API int rns_linear_small(const void* d_x, int x_type, int m, int k, int64_t ldx, int per_row,
                             const int8_t* d_w_packed, int n, const int32_t* moduli, int channels,
                             const float* d_col_scale, const float* d_bias, void* d_out, int64_t ldo,
                             int32_t out_type, rns_stream_t stream);

/*
 * Few tokens on LARGE weights (decode steps of a big model: M <= 64, any K % 16 == 0, 2..5
 * channels): the same result as rns_linear_fused from ONE launch that streams the packed
 * weight once, from activations that are already quantised - d_q int8 [M,K] (row stride ldq,
 * a multiple of 8; 8-byte aligned) with their scale(s) on the device, as
 * rns_quantize_activations leaves them (plain layout).  Floating outputs:
 * type(f32(x) * d_row_scale[m * row_scale_stride] * d_col_scale[n] (+ d_bias[n])); integer
 * outputs (d_row_scale NULL): the exact products.  No scratch.  No counterpart in the
 * reference, whose path is the same for every M (layers/rns_linear.py:237-275).
 */
RNS_API int rns_linear_stream_supported(int m, int k, int channels);
RNS_API int rns_linear_stream(const int8_t* d_q, int m, int k, int64_t ldq, const float* d_row_scale,
                              int row_scale_stride, const int8_t* d_w_packed, int n,
                              const int32_t* moduli, int channels, const float* d_col_scale,
                              const float* d_bias, void* d_out, int64_t ldo, int32_t out_type,
                              rns_stream_t stream);

/*
 * The floating-point linear for hosts that cannot allocate device memory.  It
 * has no counterpart in the reference, whose workspaces are torch tensors.
 *
 * Who needs it: a C or C++ serving loop that binds this library through the C
 * ABI, is handed its input and output buffers by its own framework, and must
 * not call cudaMalloc on the request path (it may own no allocator at all).
 * The two-step path above asks such a caller for scratch it does not have - the
 * quantised activations, their scale and a reduction word.  Here that scratch
 * is a fixed array inside the library, RNS_STATIC_SCRATCH_BYTES of packed
 * activations plus a 256-byte control block, present on every GPU that loads
 * the library until the process exits.
 *
 *   y[M,N] = type( f32(q(x) . Wq^T) * s_a * col_scale[n] + bias[n] ),
 *   q, s_a = per-tensor symmetric 8-bit quantisation of x, as RNSLinear.forward.
 *
 * d_x is [M,K] of `type` (row stride ldx elements); d_w_packed comes from
 * rns_pack_weight; d_out is [M,N] of out_type (F16/BF16/F32, row stride ldo).
 * Problems whose packed activations (rns_packed_activation_bytes(m, k, 1)) do
 * not fit the array are refused with RNS_ERR_UNSUPPORTED.
 *
 * The first call on each device looks up the array's device address, with that
 * device current; make that first call before starting any stream capture.  No
 * call allocates or frees.  Every call uses the same array: the quantiser clears
 * the one word that must start at zero, everything else is overwritten before it
 * is read, and two calls whose work overlaps on the GPU (different streams)
 * would race - serialise them.
 */
#define RNS_STATIC_SCRATCH_BYTES (8u << 20)
RNS_API int64_t rns_static_scratch_bytes(void);
RNS_API int rns_linear_static(const void* d_x, rns_float_type type, int m, int k, int64_t ldx,
                              const int8_t* d_w_packed, int n, const int32_t* moduli, int channels,
                              const float* d_col_scale, const float* d_bias, void* d_out, int64_t ldo,
                              int32_t out_type, int32_t* d_status, rns_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* RNS_B200_H_ */
