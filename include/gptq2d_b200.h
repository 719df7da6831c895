/*
 * gptq2d_b200 -- C ABI of the B200 (sm_100a) GPTQ-2D rounding engine.
 *
 * Every entry point is extern "C", takes plain device pointers and sizes,
 * launches its kernels asynchronously on the CUDA stream it is given, never
 * allocates device memory, never synchronizes and never reads device memory
 * from the host, so a call can be captured in a CUDA graph.  Buffers are owned
 * by the caller.  Two exceptions, both one-time set-up: the first call of a kernel
 * on a device sets a function attribute, and the first g2d_sweep_fused call on a
 * device that takes the pipelined schedule creates the library's side streams and
 * events; make those first calls outside stream capture (inside a capture the
 * latter returns G2D_ERR_UNSUPPORTED instead).  Calls are safe from several host
 * threads; work given to one stream is ordered as issued.
 * Return value: 0 (G2D_OK) or a negative g2d_status; g2d_status_string names it.
 *
 * Each declaration cites the function of the reference (IST-DASLab/GPTQ-2D,
 * file:line within that project) whose work it replaces.
 */
#ifndef GPTQ2D_B200_H
#define GPTQ2D_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum g2d_status {
    G2D_OK = 0,
    G2D_ERR_BAD_ARGUMENT = -1,   /* a size, stride, enum or pointer is invalid */
    G2D_ERR_WORKSPACE = -2,      /* workspace pointer missing or too small */
    G2D_ERR_UNSUPPORTED = -3,    /* a combination this build does not implement */
    G2D_ERR_CUDA = -4,           /* a CUDA runtime call failed (launch, attribute) */
    G2D_ERR_TOO_LARGE = -5       /* a size exceeds a documented fixed maximum */
} g2d_status;

typedef enum g2d_dtype { G2D_F32 = 0, G2D_F64 = 1 } g2d_dtype;
typedef enum g2d_half { G2D_FP16 = 0, G2D_BF16 = 1 } g2d_half;

typedef enum g2d_quant_kind {
    G2D_Q_ROUND = 0,   /* quantizer_int.py:18-35  round half to even */
    G2D_Q_AFFINE = 1,  /* quantizer_int.py:63-107 (clamp(rint(y/scale + zp), qmin, qmax) - zp) * scale */
    G2D_Q_ABSMAX_DYNAMIC = 2, /* quantizer_int.py:120-134 every row of a super-entry rounded under its own abs-max scale (g2d_sweep_super_entry) */
    G2D_Q_TRELLIS = 3, /* quantizer_trellis.py:344-391 every super-entry a bitshift-trellis sequence (g2d_sweep_super_entry) */
    G2D_Q_FORCED = 4   /* commit the given values (teacher-forced replay for parity checks) */
} g2d_quant_kind;

/* One batched sweep problem.  Matrices are row-major; batch b of a [batch, m, n]
 * buffer starts b*m*n elements in.  L, U, scale and zero point are addressed as
 * base + offsets[b] (element offsets, device array of `batch` int64) so that
 * broadcast batch dimensions are not copied; a NULL offsets pointer means 0. */
typedef struct g2d_sweep_desc {
    int32_t dtype;               /* g2d_dtype shared by every floating-point buffer */
    int32_t quant_kind;          /* g2d_quant_kind */
    int64_t batch, m, n;
    void *y;                     /* [batch, m, n]: X on entry, Z on return */
    const void *l;               /* [.., m, m] unit lower; read only strictly below the diagonal */
    const int64_t *l_offsets;
    const void *u;               /* [.., n, n] unit upper; read only strictly above the diagonal */
    const int64_t *u_offsets;
    const void *scale;           /* AFFINE: [.., m, n] through (scale_row_stride, scale_col_stride) */
    const int64_t *scale_offsets;
    const void *zero;            /* AFFINE: zero points, same addressing with its own strides */
    const int64_t *zero_offsets;
    int64_t scale_row_stride, scale_col_stride, zero_row_stride, zero_col_stride;
    double qmin, qmax;           /* AFFINE clamp; +-infinity disables it */
    const void *forced_z;        /* FORCED: [batch, m, n] values to commit */
    void *y_pre;                 /* optional [batch, m, n]: every entry's value when it was rounded */
    void *workspace;             /* g2d_sweep_workspace_bytes() bytes, 256-byte aligned */
    size_t workspace_bytes;
    int32_t outer_tiles;         /* tile anti-diagonals per far update; 0 selects the default */
    int32_t reserved;            /* launch schedule: 0 library default, 1 tile, 2 macro, 3 pipelined schedule */
    int32_t *status;             /* optional device int32: set to -1 when a bounded wait inside a tensor-core update kernel
                                    ran out (the kernels never spin without limit).  Y is then overwritten with NaN as well,
                                    so such a sweep cannot be mistaken for a result.  Never cleared by the library. */
} g2d_sweep_desc;

const char *g2d_status_string(int status);
/* ABI version of this header: bumped whenever a struct or signature changes. */
int g2d_abi_version(void);

/* Fused tile-wavefront sweep with the quantizer inside the kernels.
 * Replaces gptq_2d (gptq_2d.py:1379-1418) = _gptq_2d_blocked (:1295-1375) with its per-stage
 * quantizer call and the kernels _push_kernel (:243), _add_own_errors_kernel (:381),
 * _repack_errors_kernel (:632), _flush_down_kernel (:765), _flush_right_kernel (:935),
 * for quantizers this library knows: round_quantizer (quantizer_int.py:18) and
 * affine_quantizer_torch/_triton (quantizer_int.py:63, :208). */
int g2d_sweep_workspace_bytes(const g2d_sweep_desc *desc, size_t *bytes);
int g2d_sweep_fused(const g2d_sweep_desc *desc, void *stream);

/* g2d_sweep_fused for callers that cannot allocate device memory (no counterpart in the reference, whose
 * Python driver always allocates its buffers with torch).  Meant for a plugin inside a host application that
 * has reserved the whole device and offers no allocator, or for a latency-bound service that must not call
 * cudaMalloc (a device-wide synchronisation) while running: the caller passes inputs and outputs only
 * (desc->workspace and desc->workspace_bytes are ignored) and the two scratch planes come from a fixed
 * G2D_STATIC_SCRATCH_BYTES array that each device holds from library load to process exit.
 *  - Limit: g2d_sweep_workspace_bytes(desc) <= G2D_STATIC_SCRATCH_BYTES, i.e. batch*m*n <= 4 Mi fp32 or 2 Mi fp64
 *    elements (2048 x 2048 fp32); larger problems return G2D_ERR_TOO_LARGE ("size exceeds a fixed maximum").
 *  - The first call on each device looks up the array's device address (with that device current); make that
 *    first call before any stream capture begins.
 *  - All calls on a device share the array, which keeps the previous call's contents (the sweep clears what it
 *    needs cleared).  Two calls that overlap on the GPU, e.g. on different streams, race: serialise them.
 *  - Calls no cudaMalloc / cudaFree and no allocating library routine.  It always takes the tile schedule, so its
 *    results are those of g2d_sweep_fused with desc->reserved = 1, bit for bit (for one fp32 matrix whose sides are
 *    multiples of 4, g2d_sweep_fused by default takes the pipelined schedule, which sums the feedback in another
 *    order and may differ at rounding ties). */
#define G2D_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)
int g2d_sweep_fused_static(const g2d_sweep_desc *desc, void *stream);

/* A sweep over p x q super-entries, or an N-factor sweep, with the quantizer inside the library: the whole loop over the
 * coarse anti-diagonals runs inside the call (quantizer kernel, commit and in-block pushes, block-end updates), where the
 * reference's Python driver makes several launches per stage from the host.
 * Replaces gptq_2d_super_entry (gptq_2d.py:1422-1447) = _gptq_2d_blocked (:1295-1375) with _push_down_super_entry_kernel
 * (:428-505), _push_right_super_entry_kernel (:536-601) and _flush_block (:1090-1119), for the quantizers
 * round_quantizer_super_entry (quantizer_int.py:28), affine_quantizer_super_entry_* (:86, :302), int_abs_max_quantizer_*
 * (:120, :442) and trellis_quantizer_super_entry_* (quantizer_trellis.py:344, :372); and, with lead_count > 0,
 * alg4 (gptq_2d_reference.py:269-294): the tensor [lead_size[0], .., lead_size[lead_count-1], m, n] with one unit lower
 * triangular factor per leading mode (lead_factor[k], row-major [size, size], read strictly below the diagonal), l for
 * mode m and u (upper, = the last mode's factor transposed) for mode n.  The leading factors are applied mode by mode;
 * no Kronecker product is formed.  y is then [batch = product of lead_size, m, n] and the super-entry is (1, .., 1, p, q). */
typedef struct g2d_super_desc {
    int32_t dtype;               /* g2d_dtype */
    int32_t quant_kind;          /* ROUND, AFFINE, ABSMAX_DYNAMIC or TRELLIS */
    int32_t p, q;                /* super-entry shape; must divide m and n */
    int32_t inner_block, outer_block; /* coarse stages per inner / outer block, clamped as gptq_2d.py:1327-1329 does (<= 0: one block) */
    int64_t batch, m, n;
    void *y;                     /* [batch, m, n]: X on entry, Z on return */
    const void *l;               /* [.., m, m]: read only below the p x p diagonal blocks */
    const int64_t *l_offsets;    /* per-batch element offsets as in g2d_sweep_desc; NULL = 0 */
    const void *u;               /* [.., n, n]: read only above the q x q diagonal blocks */
    const int64_t *u_offsets;
    int32_t lead_count;          /* 0 for a two-sided sweep; else the number of leading modes (<= 4) */
    int32_t half;                /* ABSMAX_DYNAMIC: g2d_half of the scale */
    int64_t lead_size[4];
    const void *lead_factor[4];
    const void *scale;           /* AFFINE: [.., m, n] through the strides below; TRELLIS: one value per batch (scale_offsets) */
    const int64_t *scale_offsets;
    const void *zero;            /* AFFINE */
    const int64_t *zero_offsets;
    int64_t scale_row_stride, scale_col_stride, zero_row_stride, zero_col_stride;
    double qmin, qmax;           /* AFFINE, ABSMAX_DYNAMIC */
    const void *table;           /* TRELLIS: [2^L, V] in dtype; a super-entry read row by row is one sequence of p q values */
    int32_t trellis_L, trellis_K, trellis_V, tail_biting;
    uint8_t *codes;              /* TRELLIS, optional: packed paths, [batch, m / p, n / q, g2d_trellis_code_bytes] */
    void *workspace;             /* g2d_super_workspace_bytes() bytes, 256-byte aligned */
    size_t workspace_bytes;
    const void *table_distinct;  /* TRELLIS, optional index of the table (see g2d_trellis_quantize_indexed): its distinct rows, */
    const uint16_t *table_ids;   /* the row number of every state among them (16-byte aligned), */
    int32_t table_distinct_count; /* and how many there are */
    int32_t reserved;            /* must be 0 */
} g2d_super_desc;
int g2d_super_workspace_bytes(const g2d_super_desc *desc, size_t *bytes);
int g2d_sweep_super_entry(const g2d_super_desc *desc, void *stream);

/* Profiling variant of g2d_sweep_fused (no counterpart in the reference): the same launches, each
 * bracketed by a CUDA event pair on `stream`; synchronizes the stream before returning, so it cannot be
 * captured.  out[0..2] = total milliseconds of the tile-sweep / near-update / far-update launches,
 * out[3..5] = their launch counts, out[6] = algorithmic flops of the whole sweep m n (m + n - 2) per
 * batch, out[7], out[8] = algorithmic flops executed by the near / far updates. */
int g2d_sweep_fused_profile(const g2d_sweep_desc *desc, void *stream, double *out);

/* Kernel launches made by this library in this process so far (host-side counter). */
unsigned long long g2d_launch_count(void);

/* Generic per-stage path: the caller's own quantizer runs between these calls, one coarse
 * anti-diagonal (stage) at a time, and sees live Y as the reference promises (gptq_2d.py:1395-1400).
 * Geometry shared by the three calls. y, c, e are [batch, m, n]; c must start at zero. */
typedef struct g2d_stage_desc {
    int32_t dtype;
    int32_t p, q;                /* super-entry shape; 1, 1 for plain entries */
    int32_t reserved;            /* must be 0 */
    int64_t batch, m, n;
    void *y;                     /* live Y (X plus every push so far; quantized where done) */
    void *c;                     /* running buffer C = L E (gptq_2d.py:1324) */
    void *e;                     /* errors E of every finished entry, natural [batch, m, n] layout */
    const void *l;
    const int64_t *l_offsets;
    const void *u;
    const int64_t *u_offsets;
} g2d_stage_desc;

/* Stage s of the block [.., s1): take the quantized values z ([batch, d, p, q] contiguous, d the
 * number of super-entries of the stage), form E = z - Y, complete C on the sources, commit Y = z,
 * and push the errors down through L and the completed C right through U to the stages s+1..s1-1.
 * Replaces _push_kernel (gptq_2d.py:243-346) + _add_own_errors_kernel (:381-409) for plain entries and
 * _push_down_super_entry_kernel (:428-505) + _push_right_super_entry_kernel (:536-601) otherwise. */
int g2d_stage_push(const g2d_stage_desc *desc, const void *z, int64_t s, int64_t s1, void *stream);

/* Apply the errors of the stages s0..s1-1 to the stages s1..s_end-1: C += L E and Y += L E + C U with
 * the sums restricted to the sources of those stages.  Replaces _flush_block (gptq_2d.py:1090-1119) =
 * _repack_errors_kernel (:632) + _flush_down_kernel (:765) + _flush_right_kernel (:935). */
int g2d_stage_flush(const g2d_stage_desc *desc, int64_t s0, int64_t s1, int64_t s_end, void *stream);

/* Strided affine quantizer: out[b, k] = affine(y[b*matrix_size + start + k*step]) for k < count, with
 * scale / zero point read at the same position of their own matrices (base + offsets[b]).
 * Replaces _affine_quantize_kernel (quantizer_int.py:160-205). */
int g2d_affine_quantize(int dtype, int64_t batch, int64_t matrix_size, int64_t start, int64_t step, int64_t count,
                        const void *y, const void *scale, const int64_t *scale_offsets, const void *zero,
                        const int64_t *zero_offsets, double qmin, double qmax, void *out, void *stream);

/* Super-entry affine quantizer: entry (k, r, c) of the selection lies k*stride_d + r*stride_p + c*stride_q
 * past `first` in Y, scale and zero point alike; out is [batch, d, p, q] contiguous.
 * Replaces _affine_quantize_super_entry_kernel (quantizer_int.py:247-299). */
int g2d_affine_quantize_super_entry(int dtype, int64_t batch, int64_t matrix_size, int64_t first, int64_t d, int32_t p,
                                    int32_t q, int64_t stride_d, int64_t stride_p, int64_t stride_q, const void *y,
                                    const void *scale, const int64_t *scale_offsets, const void *zero,
                                    const int64_t *zero_offsets, double qmin, double qmax, void *out, void *stream);

/* Row scales absmax / ((qmax - qmin) / 2), rounded to fp16 / bf16 through fp32, 0 -> 1.
 * Replaces _int_abs_max_scale_kernel (quantizer_int.py:357-385). */
int g2d_absmax_scale(int dtype, int64_t rows, int64_t size, int64_t row_stride, int64_t col_stride, const void *x,
                     double qmin, double qmax, int half, void *out, void *stream);

/* Dynamic abs-max rounding of every row of the selected super-entries.
 * Replaces _int_abs_max_quantize_kernel (quantizer_int.py:407-439). */
int g2d_absmax_quantize_super_entry(int dtype, int64_t batch, int64_t matrix_size, int64_t first, int64_t d, int32_t p,
                                    int32_t q, int64_t stride_d, int64_t stride_p, int64_t stride_q, const void *y,
                                    double qmin, double qmax, int half, void *out, void *stream);

/* Bitshift-trellis (Viterbi) search of `rows` sequences of T values: out = scale[row] * values of the
 * closest path, states optional ([rows, T/V] int64).  table is [2^L, V] in dtype, V <= 2, K*V <= 8.
 * workspace: g2d_trellis_workspace_bytes().  Replaces _viterbi_step_kernel, _viterbi_final_kernel and
 * _viterbi_backtrack_kernel (quantizer_trellis.py:146-268) as driven by _trellis_quantize_triton (:271-341). */
int g2d_trellis_workspace_bytes(int dtype, int64_t rows, int32_t T, int32_t L, int32_t K, int32_t V, size_t *bytes);
int g2d_trellis_quantize(int dtype, int64_t rows, int32_t T, const void *x, const void *table, int32_t L, int32_t K,
                         int32_t V, int32_t tail_biting, const void *scale, void *out, int64_t *states,
                         void *workspace, size_t workspace_bytes, void *stream);

/* The same search that also stores every path as its bit string, the storage format of a trellis code (the reference
 * only notes that "the T K-bit code can be recovered" from the values, quantizer_trellis.py:11-14).  The string holds the
 * K V bits that each step shifts into the state, most significant bit first, preceded, unless the path is tail-biting,
 * by the L - K V upper bits of the first state; bit i of the string is bit i % 8 of byte i / 8, and a sequence takes
 * g2d_trellis_code_bytes bytes (T K / 8 when tail-biting).  g2d_trellis_decode turns strings back into scale * values
 * (and the int64 states, optional), bit for bit what the search returned. */
int g2d_trellis_code_bytes(int32_t T, int32_t L, int32_t K, int32_t V, int32_t tail_biting, int64_t *bytes);
int g2d_trellis_quantize_packed(int dtype, int64_t rows, int32_t T, const void *x, const void *table, int32_t L, int32_t K,
                                int32_t V, int32_t tail_biting, const void *scale, void *out, uint8_t *codes,
                                void *workspace, size_t workspace_bytes, void *stream);
int g2d_trellis_decode(int dtype, int64_t rows, int32_t T, const uint8_t *codes, const void *table, int32_t L, int32_t K,
                       int32_t V, int32_t tail_biting, const void *scale, void *out, int64_t *states, void *stream);

/* The same search for a caller who knows which states of the table share their values.  The shipped codes map 2^16
 * states onto about a thousand distinct value tuples (hyb: quantizer_trellis.py:63-79, a 2^9-row lookup table times a
 * sign; one_mad: :28-33, a sum of four bytes), and a state's local cost depends on its tuple only.  `distinct` holds the
 * distinct rows of `table` ([distinct_count, V], same dtype) and `ids[s]` the row of state s among them; tables of up to
 * 2^16 states whose distinct rows fit shared memory are then searched from shared memory, others as by
 * g2d_trellis_quantize.  Values, states and stored paths (states, codes: optional) are bit for bit the same. */
int g2d_trellis_quantize_indexed(int dtype, int64_t rows, int32_t T, const void *x, const void *table, int32_t L, int32_t K,
                                 int32_t V, int32_t tail_biting, const void *scale, void *out, int64_t *states, uint8_t *codes,
                                 const void *distinct, int32_t distinct_count, const uint16_t *ids, void *workspace,
                                 size_t workspace_bytes, void *stream);

/* Unit (block) lower triangular factor of the inverse of a symmetric positive definite matrix:
 * a^{-1} = out Lambda out^T with size x size identity diagonal blocks.  a is [n, n] and is overwritten
 * (scratch); workspace: g2d_ldl_workspace_bytes().  status_flag (device int32, may be NULL) receives the
 * 1-based index of a non-positive pivot, or stays 0.
 * Replaces ldl_of_inverse (gptq_2d_reference.py:41-49) with _unit_diagonal_blocks (:29-38). */
int g2d_ldl_workspace_bytes(int dtype, int64_t n, size_t *bytes);
int g2d_ldl_of_inverse(int dtype, int64_t n, void *a, int32_t size, void *out, int32_t *status_flag, void *workspace,
                       size_t workspace_bytes, void *stream);

/* Two factorizations of g2d_ldl_of_inverse advanced together in the same launches (both are chains of short
 * dependent kernels, so the pair costs little more than the larger one): the L and U of one layer, i.e. both
 * calls of feedback_factors (gptq_2d_reference.py:52-66).  Each problem has its own workspace
 * (g2d_ldl_workspace_bytes of its n); status_flags is int32[2] on the device or NULL.  Results are identical
 * to two single calls. */
int g2d_ldl_of_inverse_pair(int dtype, int64_t n0, void *a0, int32_t size0, void *out0, void *workspace0,
                            size_t workspace0_bytes, int64_t n1, void *a1, int32_t size1, void *out1,
                            void *workspace1, size_t workspace1_bytes, int32_t *status_flags, void *stream);

/* Hessian-factor accumulation h += alpha * x^T x on the tensor cores: x is [k samples, n channels] float, h is
 * [n, n] float (both row-major, n a multiple of 4).  No counterpart in the reference, which takes its Hessian
 * factors from the caller (demo.ipynb:103-106 forms them with a plain matrix product); it is the step before
 * g2d_ldl_of_inverse in a pipeline.  workspace: g2d_gram_workspace_bytes(); status_flag (device int32, may be
 * NULL) is set to -1 if a bounded wait inside the kernel ran out. */
int g2d_gram_workspace_bytes(int64_t n, int64_t k, size_t *bytes);
int g2d_gram_accumulate(int64_t n, int64_t k, const float *x, float alpha, float *h, int32_t *status_flag,
                        void *workspace, size_t workspace_bytes, void *stream);

/* Packed integer codes of a rounded matrix z [m, n] and back.  The reference has no counterpart: it returns
 * dequantised floats and notes that the code can be recovered from them (quantizer_trellis.py:11-14; for the
 * affine quantizer, quantizer_int.py:63-83, code = rint(z / scale + zero point)).  Entry j of a row is the
 * `bits`-bit unsigned field code - qmin (clamped to the field) at the bits j*bits .. j*bits+bits-1 of the
 * row's byte string (little-endian); rows are row_bytes >= ceil(n*bits/8) apart.  scale and zero point are
 * addressed by row and column strides in elements (0 = broadcast).  g2d_unpack_codes forms
 * (code + qmin - zero point) * scale, the value the affine quantizer returned, bit for bit. */
int g2d_pack_codes(int dtype, int64_t m, int64_t n, const void *z, const void *scale, int64_t scale_row_stride,
                   int64_t scale_col_stride, const void *zero, int64_t zero_row_stride, int64_t zero_col_stride,
                   double qmin, int32_t bits, uint8_t *codes, int64_t row_bytes, void *stream);
int g2d_unpack_codes(int dtype, int64_t m, int64_t n, const uint8_t *codes, int64_t row_bytes, const void *scale,
                     int64_t scale_row_stride, int64_t scale_col_stride, const void *zero, int64_t zero_row_stride,
                     int64_t zero_col_stride, double qmin, int32_t bits, void *z, void *stream);

/* Full symmetric matrix out [n, n] from its packed lower triangle (row i holds the entries (i, 0 .. i); n (n + 1) / 2
 * values): the form in which a Hessian factor can travel from host memory at half the bytes.  No counterpart in the
 * reference, whose inputs are device tensors. */
int g2d_symmetric_from_packed(int dtype, int64_t n, const void *packed, void *out, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* GPTQ2D_B200_H */
