/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the GPTQ-2D rounding path.
 *
 * This header is included twice by g2d_oracle.c, once per working type
 * (REAL = float, SFX = f32; REAL = double, SFX = f64).  It restates, in plain
 * C, what the reference's PyTorch implementation computes; every function
 * names the reference file:line it follows.  It is the checker for the CUDA
 * library and the timed CPU baseline; it is never linked into the product.
 *
 * All arithmetic is done in REAL with contraction disabled (the build passes
 * -ffp-contract=off), rounding is to nearest-even, divisions are IEEE.
 */

#define CAT_(a, b) a##_##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SFX)

/* ---- elementwise quantizers ------------------------------------------- */

/* quantizer_int.py:63-83 (affine_quantizer_torch): div, add zero point,
 * round half-even, clamp, subtract zero point, multiply by scale. */
static inline REAL FN(affine_one)(REAL y, REAL scale, REAL zp, REAL qmin, REAL qmax) {
    REAL t = y / scale;
    t = t + zp;
    t = RINT(t);
    /* torch.clamp_(min, max) == min(max(t, lo), hi); NaN propagates */
    if (t < qmin) t = qmin;
    if (t > qmax) t = qmax;
    t = t - zp;
    return t * scale;
}

/* quantizer_int.py:110-117 (int_abs_max_scale_torch): absmax / ((qmax-qmin)/2)
 * rounded to a 16-bit float type through fp32, returned in REAL, 0 -> 1. */
static inline REAL FN(absmax_scale_one)(REAL absmax, double qmin, double qmax, int half_kind) {
    REAL divisor = (REAL)((qmax - qmin) / 2.0);
    REAL s = absmax / divisor;
    float f = (float)s;
    f = half_kind == G2D_ORC_BF16 ? orc_round_bf16(f) : orc_round_fp16(f);
    s = (REAL)f;
    return s == (REAL)0 ? (REAL)1 : s;
}

void FN(orc_affine_quantize)(int64_t count, const REAL *y, const REAL *scale, const REAL *zp,
                             double qmin, double qmax, REAL *out) {
    for (int64_t k = 0; k < count; ++k)
        out[k] = FN(affine_one)(y[k], scale[k], zp[k], (REAL)qmin, (REAL)qmax);
}

/* rows of `size` entries, entry c of row r at x[r*row_stride + c*col_stride] */
void FN(orc_absmax_scale)(int64_t rows, int64_t size, const REAL *x, int64_t row_stride, int64_t col_stride,
                          double qmin, double qmax, int half_kind, REAL *out) {
    for (int64_t r = 0; r < rows; ++r) {
        REAL a = 0;
        for (int64_t c = 0; c < size; ++c) {
            REAL v = FABS(x[r * row_stride + c * col_stride]);
            if (v > a) a = v;
        }
        out[r] = FN(absmax_scale_one)(a, qmin, qmax, half_kind);
    }
}

/* quantizer_int.py:120-134 (int_abs_max_quantizer_torch) on one row of q entries */
static inline void FN(absmax_quantize_row)(int q, const REAL *y, int64_t stride, double qmin, double qmax,
                                           int half_kind, REAL *out) {
    REAL a = 0;
    for (int c = 0; c < q; ++c) {
        REAL v = FABS(y[c * stride]);
        if (v > a) a = v;
    }
    REAL s = FN(absmax_scale_one)(a, qmin, qmax, half_kind);
    for (int c = 0; c < q; ++c) {
        REAL t = RINT(y[c * stride] / s);
        if (t < (REAL)qmin) t = (REAL)qmin;
        if (t > (REAL)qmax) t = (REAL)qmax;
        out[c] = t * s;
    }
}

/* ---- trellis (Viterbi) -------------------------------------------------- */

/* quantizer_trellis.py:82-118 (_viterbi) for one sequence.
 * x: [steps*V]; roll: read step t from x[((t + roll) % steps)*V ...].
 * init_overlap >= 0 restricts the first state to (s >> shift) == init_overlap,
 * final_overlap >= 0 restricts the last state to (s mod G) == final_overlap.
 * cost/next: scratch [S]; choices: scratch [(steps-1)*G] bytes (shift <= 8) */
static void FN(viterbi_one)(const REAL *x, int steps, int V, const REAL *table, int Lbits, int shift, int roll,
                            int64_t init_overlap, int64_t final_overlap, REAL *cost, REAL *next, REAL *best,
                            uint8_t *choices, int64_t *states) {
    const int64_t S = (int64_t)1 << Lbits, G = S >> shift, H = (int64_t)1 << shift;
    const REAL inf = (REAL)INFINITY;
    {
        const REAL *xt = x + (int64_t)((0 + roll) % steps) * V;
        for (int64_t s = 0; s < S; ++s) {
            REAL acc = 0;
            for (int v = 0; v < V; ++v) {
                REAL d = table[s * V + v] - xt[v];
                acc = v == 0 ? d * d : acc + d * d;
            }
            if (init_overlap >= 0 && (s >> shift) != init_overlap) acc = inf;
            cost[s] = acc;
        }
    }
    for (int t = 1; t < steps; ++t) {
        uint8_t *ch = choices + (int64_t)(t - 1) * G;
        for (int64_t g = 0; g < G; ++g) {
            REAL b = cost[g];
            int hb = 0;
            for (int64_t h = 1; h < H; ++h) {
                REAL c = cost[h * G + g];
                if (c < b) { b = c; hb = (int)h; }
            }
            best[g] = b;
            ch[g] = (uint8_t)hb;
        }
        const REAL *xt = x + (int64_t)((t + roll) % steps) * V;
        for (int64_t s = 0; s < S; ++s) {
            REAL acc = 0;
            for (int v = 0; v < V; ++v) {
                REAL d = table[s * V + v] - xt[v];
                acc = v == 0 ? d * d : acc + d * d;
            }
            next[s] = best[s >> shift] + acc;
        }
        REAL *tmp = cost; cost = next; next = tmp;
    }
    /* first index of the least (masked) cost */
    int64_t arg = 0;
    REAL b = (final_overlap >= 0 && (0 & (G - 1)) != final_overlap) ? inf : cost[0];
    for (int64_t s = 1; s < S; ++s) {
        REAL c = cost[s];
        if (final_overlap >= 0 && (s & (G - 1)) != final_overlap) c = inf;
        if (c < b) { b = c; arg = s; }
    }
    states[steps - 1] = arg;
    for (int t = steps - 1; t >= 1; --t) {
        int64_t low = states[t] >> shift;
        states[t - 1] = (int64_t)choices[(int64_t)(t - 1) * G + low] * G + low;
    }
}

/* quantizer_trellis.py:121-143 (_trellis_quantize_torch): rows sequences of T
 * values; values [rows*T] and states [rows*(T/V)] out (states may be NULL). */
int FN(orc_trellis_quantize)(int64_t rows, int T, const REAL *x, const REAL *table, int Lbits, int K, int V,
                             int tail_biting, REAL *values, int64_t *states_out) {
    const int shift = K * V, steps = T / V;
    if (shift > 8 || shift > Lbits || T % V != 0 || steps < 1) return -1;
    const int64_t S = (int64_t)1 << Lbits, G = S >> shift;
    int status = 0;
#pragma omp parallel
    {
        REAL *cost = (REAL *)malloc(sizeof(REAL) * S), *next = (REAL *)malloc(sizeof(REAL) * S);
        REAL *best = (REAL *)malloc(sizeof(REAL) * G);
        uint8_t *choices = (uint8_t *)malloc((size_t)(steps > 1 ? steps - 1 : 1) * G);
        int64_t *st = (int64_t *)malloc(sizeof(int64_t) * steps);
        if (!cost || !next || !best || !choices || !st) {
#pragma omp atomic write
            status = -2;
        } else {
#pragma omp for schedule(dynamic, 1)
            for (int64_t r = 0; r < rows; ++r) {
                const REAL *xr = x + r * T;
                int64_t overlap = -1;
                if (tail_biting) {
                    int half = steps / 2;
                    /* x.roll(half*V): rolled step t reads original step (t - half) mod steps */
                    FN(viterbi_one)(xr, steps, V, table, Lbits, shift, steps - half, -1, -1, cost, next, best, choices, st);
                    overlap = st[half] >> shift;
                }
                FN(viterbi_one)(xr, steps, V, table, Lbits, shift, 0, overlap, overlap, cost, next, best, choices, st);
                for (int t = 0; t < steps; ++t) {
                    for (int v = 0; v < V; ++v) values[r * T + t * V + v] = table[st[t] * V + v];
                    if (states_out) states_out[r * steps + t] = st[t];
                }
            }
        }
        free(cost); free(next); free(best); free(choices); free(st);
    }
    return status;
}

/* ---- the sweep ------------------------------------------------------------ */

typedef struct {
    int kind;              /* G2D_ORC_Q_* */
    double qmin, qmax;     /* affine / absmax clamp */
    const REAL *scale;     /* affine: [m*n]; trellis: [1] scalar scale */
    const REAL *zero;      /* affine: [m*n] */
    int half_kind;         /* absmax: fp16 / bf16 */
    const REAL *table;     /* trellis: [2^L * V] */
    int Lbits, K, V, tail_biting;
    const REAL *forced_z;  /* FORCED: [m*n] values to commit */
    REAL *y_pre;           /* optional [m*n]: value of every entry when it was rounded */
} FN(orc_quant);

/* gptq_2d.py:1240-1292 (gptq_2d_super_entry_torch; p = q = 1 is gptq_2d_torch,
 * gptq_2d.py:1197-1236): anti-diagonal sweep over the coarse (m/p) x (n/q)
 * grid of p x q super-entries.  y holds X on entry and Z on return. L and U
 * are read only strictly below / above their p x p / q x q diagonal blocks. */
int FN(orc_sweep)(int64_t m, int64_t n, int p, int q, REAL *y, const REAL *l, const REAL *u,
                  const FN(orc_quant) *qz) {
    if (m == 0 || n == 0) return 0;
    if (p <= 0 || q <= 0 || m % p || n % q) return -1;
    const int64_t mbar = m / p, nbar = n / q, lanes = mbar < nbar ? mbar : nbar;
    const int pq = p * q;
    REAL *c = (REAL *)calloc((size_t)m * n, sizeof(REAL));
    REAL *e = (REAL *)malloc(sizeof(REAL) * lanes * pq);   /* errors of the stage, [d][p][q] */
    REAL *z = (REAL *)malloc(sizeof(REAL) * lanes * pq);
    REAL *cs = (REAL *)malloc(sizeof(REAL) * lanes * pq);  /* completed C of the sources */
    REAL *seq = (REAL *)malloc(sizeof(REAL) * lanes * pq);
    if (!c || !e || !z || !cs || !seq) { free(c); free(e); free(z); free(cs); free(seq); return -2; }
    int status = 0;
    for (int64_t s = 0; s < mbar + nbar - 1 && status == 0; ++s) {
        const int64_t i_lo = s - nbar + 1 > 0 ? s - nbar + 1 : 0, i_hi = s + 1 < mbar ? s + 1 : mbar;
        const int64_t d = i_hi - i_lo;
        /* 1. quantize the selected super-entries: z[k][a][b] */
        if (qz->kind == G2D_ORC_Q_TRELLIS) {
            /* quantizer_trellis.py:344-369: x = select(y)/scale, one sequence per super-entry row by row */
            const REAL sc = qz->scale[0];
            for (int64_t k = 0; k < d; ++k)
                for (int a = 0; a < p; ++a)
                    for (int b = 0; b < q; ++b)
                        seq[(k * p + a) * q + b] = y[((i_lo + k) * p + a) * n + (s - i_lo - k) * q + b] / sc;
            status = FN(orc_trellis_quantize)(d, pq, seq, qz->table, qz->Lbits, qz->K, qz->V, qz->tail_biting, z, NULL);
            for (int64_t k = 0; k < d * pq; ++k) z[k] = z[k] * sc;
        } else {
#pragma omp parallel for schedule(static) if (d * pq > 4096)
            for (int64_t k = 0; k < d; ++k) {
                const int64_t i0 = (i_lo + k) * p, j0 = (s - i_lo - k) * q;
                for (int a = 0; a < p; ++a) {
                    const REAL *yr = y + (i0 + a) * n + j0;
                    REAL *zr = z + (k * p + a) * q;
                    switch (qz->kind) {
                    case G2D_ORC_Q_ROUND:
                        for (int b = 0; b < q; ++b) zr[b] = RINT(yr[b]);
                        break;
                    case G2D_ORC_Q_AFFINE:
                        for (int b = 0; b < q; ++b)
                            zr[b] = FN(affine_one)(yr[b], qz->scale[(i0 + a) * n + j0 + b], qz->zero[(i0 + a) * n + j0 + b],
                                                   (REAL)qz->qmin, (REAL)qz->qmax);
                        break;
                    case G2D_ORC_Q_ABSMAX:
                        FN(absmax_quantize_row)(q, yr, 1, qz->qmin, qz->qmax, qz->half_kind, zr);
                        break;
                    case G2D_ORC_Q_FORCED:
                        for (int b = 0; b < q; ++b) zr[b] = qz->forced_z[(i0 + a) * n + j0 + b];
                        break;
                    default:
                        for (int b = 0; b < q; ++b) zr[b] = yr[b];
                    }
                }
            }
        }
        if (status) break;
        /* 2. errors e = z - y (gptq_2d.py:1283) */
        for (int64_t k = 0; k < d; ++k) {
            const int64_t i0 = (i_lo + k) * p, j0 = (s - i_lo - k) * q;
            for (int a = 0; a < p; ++a)
                for (int b = 0; b < q; ++b) {
                    const REAL yv = y[(i0 + a) * n + j0 + b];
                    if (qz->y_pre) qz->y_pre[(i0 + a) * n + j0 + b] = yv;
                    e[(k * p + a) * q + b] = z[(k * p + a) * q + b] - yv;
                }
        }
        /* 3. down: C[r, band(jbar)] += L[r, band(ibar)] @ E, same into Y (gptq_2d.py:1286-1288).
         * Rows of the own band see the identity block; rows above it see zeros. */
        const int64_t r_begin = i_lo * p;
#pragma omp parallel for schedule(static) if ((m - r_begin) * d * pq > 16384)
        for (int64_t r = r_begin; r < m; ++r) {
            const int64_t rbar = r / p;
            /* sources with ibar <= rbar reach row r */
            const int64_t k_end = (rbar < i_hi - 1 ? rbar : i_hi - 1) - i_lo + 1;
            for (int64_t k = 0; k < k_end; ++k) {
                const int64_t ibar = i_lo + k, j0 = (s - ibar) * q;
                const REAL *ek = e + k * pq;
                if (ibar == rbar) {
                    const int a = (int)(r - rbar * p);
                    for (int b = 0; b < q; ++b) {
                        c[r * n + j0 + b] += ek[a * q + b];
                        y[r * n + j0 + b] += ek[a * q + b];
                    }
                } else {
                    const REAL *lr = l + r * m + ibar * p;
                    for (int b = 0; b < q; ++b) {
                        REAL upd = lr[0] * ek[b];
                        for (int a = 1; a < p; ++a) upd += lr[a] * ek[a * q + b];
                        c[r * n + j0 + b] += upd;
                        y[r * n + j0 + b] += upd;
                    }
                }
            }
        }
        /* 4. right: Y[band(ibar), col] += C[band(ibar), band(jbar)] @ U[band(jbar), col] for columns
         * right of the source's band (gptq_2d.py:1290); the source itself is overwritten by z next. */
        for (int64_t k = 0; k < d; ++k) {
            const int64_t i0 = (i_lo + k) * p, j0 = (s - i_lo - k) * q;
            for (int a = 0; a < p; ++a)
                for (int b = 0; b < q; ++b) cs[(k * p + a) * q + b] = c[(i0 + a) * n + j0 + b];
        }
#pragma omp parallel for schedule(static) if (d * p * n > 16384)
        for (int64_t ka = 0; ka < d * p; ++ka) {
            const int64_t k = ka / p;
            const int a = (int)(ka - k * p);
            const int64_t i0 = (i_lo + k) * p, j0 = (s - i_lo - k) * q;
            REAL *yr = y + (i0 + a) * n;
            const REAL *ck = cs + (k * p + a) * q;
            for (int b = 0; b < q; ++b) {
                const REAL cv = ck[b];
                const REAL *ur = u + (j0 + b) * n;
                for (int64_t col = j0 + q; col < n; ++col) yr[col] += cv * ur[col];
            }
        }
        /* 5. commit (gptq_2d.py:1291) */
        for (int64_t k = 0; k < d; ++k) {
            const int64_t i0 = (i_lo + k) * p, j0 = (s - i_lo - k) * q;
            for (int a = 0; a < p; ++a)
                for (int b = 0; b < q; ++b) y[(i0 + a) * n + j0 + b] = z[(k * p + a) * q + b];
        }
    }
    free(c); free(e); free(z); free(cs); free(seq);
    return status;
}

/* ---- factor prep ------------------------------------------------------------ */

/* gptq_2d_reference.py:41-49 (ldl_of_inverse) with :29-38 (_unit_diagonal_blocks).
 * a: symmetric positive definite [n*n]; out: unit (block) lower triangular with
 * a^{-1} = out Lambda out^T.  work: [2*n*n] scratch.  Returns the 1-based index
 * of a non-positive pivot, 0 on success. */
int FN(orc_ldl_of_inverse)(int64_t n, const REAL *a, int size, REAL *out, REAL *work) {
    REAL *um = work;           /* upper, a = um um^T */
    REAL *inv = work + n * n;  /* um^{-1}, upper */
    memset(um, 0, sizeof(REAL) * n * n);
    /* reverse-order Cholesky: column j of um from the last to the first;
     * a[i][j] = sum_{k >= max(i,j)} um[i][k] um[j][k] */
    for (int64_t j = n - 1; j >= 0; --j) {
        REAL dsum = a[j * n + j];
        for (int64_t k = j + 1; k < n; ++k) dsum -= um[j * n + k] * um[j * n + k];
        if (!(dsum > 0)) return (int)(j + 1);
        const REAL dj = SQRT(dsum);
        um[j * n + j] = dj;
#pragma omp parallel for schedule(static) if (j > 256)
        for (int64_t i = 0; i < j; ++i) {
            REAL acc = a[i * n + j];
            const REAL *ui = um + i * n, *uj = um + j * n;
            for (int64_t k = j + 1; k < n; ++k) acc -= ui[k] * uj[k];
            um[i * n + j] = acc / dj;
        }
    }
    /* inv = um^{-1} by back substitution, one column of the identity at a time */
    memset(inv, 0, sizeof(REAL) * n * n);
#pragma omp parallel for schedule(dynamic, 8)
    for (int64_t col = 0; col < n; ++col) {
        for (int64_t i = col; i >= 0; --i) {
            REAL acc = i == col ? (REAL)1 : (REAL)0;
            const REAL *ui = um + i * n;
            for (int64_t k = i + 1; k <= col; ++k) acc -= ui[k] * inv[k * n + col];
            inv[i * n + col] = acc / ui[i];
        }
    }
    /* lower factor Lf = inv^T; normalise by its diagonal (blocks) */
    if (size == 1) {
        for (int64_t i = 0; i < n; ++i)
            for (int64_t j = 0; j < n; ++j)
                out[i * n + j] = j <= i ? inv[j * n + i] / inv[j * n + j] : (REAL)0;
        return 0;
    }
    if (n % size) return -1;
    /* out = (Lf - D) D^{-1} + I, D the lower-triangular diagonal blocks of Lf:
     * row vector x = r D^{-1} solves x D = r, by back substitution over the block's columns */
    for (int64_t i = 0; i < n; ++i) {
        for (int64_t jb = 0; jb < n / size; ++jb) {
            const int64_t j0 = jb * size;
            for (int t = size - 1; t >= 0; --t) {
                const int64_t j = j0 + t;
                if (i / size == jb) { out[i * n + j] = i == j ? (REAL)1 : (REAL)0; continue; }
                if (j0 > i) { out[i * n + j] = 0; continue; }
                REAL acc = inv[j * n + i];  /* Lf[i][j] */
                for (int t2 = t + 1; t2 < size; ++t2) acc -= out[i * n + j0 + t2] * inv[j * n + (j0 + t2)];  /* D[j0+t2][j] = Lf[j0+t2][j] */
                out[i * n + j] = acc / inv[j * n + j];
            }
        }
    }
    return 0;
}

#undef FN
#undef CAT
#undef CAT_
