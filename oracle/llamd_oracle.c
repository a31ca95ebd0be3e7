/*
 * llamd_oracle.c -- CPU restatement of the llamd reference's quantized hot path.
 *
 * THIS FILE IS TEST INFRASTRUCTURE. It is the checker the CUDA library is
 * compared against and the timed CPU baseline; the shipped library never
 * links, loads or calls it.
 *
 * Every function follows the scalar CPU path of the reference, one operation
 * at a time and in the reference's own order, because the order of the f32
 * operations is observable in the last bit. Citations are paths inside the
 * reference project.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math (see Makefile). Contraction
 * must stay off: the reference is Rust, which never fuses a*b+c.
 *
 * Third-party arithmetic that the reference reaches through dependencies:
 *   - crate `half` 2.x: `f16::from_bits(b).to_f32()` (IEEE binary16 -> binary32,
 *     exact, subnormals included). Restated in orc_f16_to_f32 as bit arithmetic.
 *   - Rust std `f32::{exp,powf,sin,cos,sqrt}`: lowered to the host libm. Here
 *     the host glibc's expf/powf/sinf/cosf/sqrtf stand in for them.
 *
 * Pinned against the reference's own unit-test vectors by tests/test_oracle_kat.py.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define QK_K 256
#define QK8_0 32
#define Q6K_BLOCK_BYTES 210
#define Q8_0_BLOCK_BYTES 34

/* ggml type ids: crates/llamd-quant/src/lib.rs:49-54 */
enum { ORC_F32 = 0, ORC_F16 = 1, ORC_Q8_0 = 8, ORC_Q6K = 14 };

/* ------------------------------------------------------------------------ */
/* f16 <-> f32                                                               */
/* ------------------------------------------------------------------------ */

/* crates/llamd-quant/src/lib.rs:104-108 (half::f16::from_bits().to_f32()) */
float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            /* subnormal: normalise */
            int e = -1;
            do {
                e++;
                man <<= 1;
            } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* half::f16::from_f32: round to nearest, ties to even. Used by the reference's
 * tests to build blocks (crates/llamd-quant/src/lib.rs:265,285). */
uint16_t orc_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t exp = (x >> 23) & 0xFFu;
    uint32_t man = x & 0x7FFFFFu;
    if (exp == 255) {
        return (uint16_t)(sign | 0x7C00u | (man ? (0x200u | (man >> 13)) : 0));
    }
    int e = (int)exp - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        man |= 0x800000u;
        int shift = 14 - e;
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1))) half_man++;
        return (uint16_t)(sign | half_man);
    }
    uint32_t half_man = man >> 13;
    uint32_t rem = man & 0x1FFFu;
    uint16_t out = (uint16_t)(sign | ((uint32_t)e << 10) | half_man);
    if (rem > 0x1000u || (rem == 0x1000u && (half_man & 1))) out++;
    return out;
}

/* ------------------------------------------------------------------------ */
/* formats                                                                   */
/* ------------------------------------------------------------------------ */

/* QuantType::block_elems / block_bytes / bytes_for:
 * crates/llamd-quant/src/lib.rs:72-101. Returns -1 for an unknown type, -2
 * for a partial block (the reference's Error::Malformed). */
int64_t orc_bytes_for(int ty, int64_t n) {
    int64_t be, bb;
    switch (ty) {
    case ORC_F32: be = 1; bb = 4; break;
    case ORC_F16: be = 1; bb = 2; break;
    case ORC_Q8_0: be = QK8_0; bb = Q8_0_BLOCK_BYTES; break;
    case ORC_Q6K: be = QK_K; bb = Q6K_BLOCK_BYTES; break;
    default: return -1;
    }
    if (n % be != 0) return -2;
    return n / be * bb;
}

static inline uint16_t rd_u16(const uint8_t *b) { return (uint16_t)(b[0] | (b[1] << 8)); }

/* crates/llamd-quant/src/lib.rs:154-162 */
static void dequantize_q8_0(const uint8_t *src, int64_t n, float *out) {
    for (int64_t b = 0; b < n / QK8_0; b++) {
        const uint8_t *blk = src + b * Q8_0_BLOCK_BYTES;
        float d = orc_f16_to_f32(rd_u16(blk));
        for (int j = 0; j < QK8_0; j++) out[b * QK8_0 + j] = d * (float)(int8_t)blk[2 + j];
    }
}

/* crates/llamd-quant/src/lib.rs:181-226 */
static void dequantize_q6_k(const uint8_t *src, int64_t n, float *out) {
    const int QL = 0, QH = QK_K / 2, SC = QK_K / 2 + QK_K / 4, D = QK_K / 2 + QK_K / 4 + QK_K / 16;
    for (int64_t b = 0; b < n / QK_K; b++) {
        const uint8_t *blk = src + b * Q6K_BLOCK_BYTES;
        float d = orc_f16_to_f32(rd_u16(blk + D));
        float *y0 = out + b * QK_K;
        for (int half = 0; half < 2; half++) {
            int ql = QL + half * 64, qh = QH + half * 32, sc = SC + half * 8;
            float *y = y0 + half * 128;
            for (int l = 0; l < 32; l++) {
                int is = l / 16;
                uint8_t h = blk[qh + l], lo0 = blk[ql + l], lo1 = blk[ql + l + 32];
                int8_t q1 = (int8_t)((lo0 & 0x0F) | (((h >> 0) & 3) << 4)) - 32;
                int8_t q2 = (int8_t)((lo1 & 0x0F) | (((h >> 2) & 3) << 4)) - 32;
                int8_t q3 = (int8_t)((lo0 >> 4) | (((h >> 4) & 3) << 4)) - 32;
                int8_t q4 = (int8_t)((lo1 >> 4) | (((h >> 6) & 3) << 4)) - 32;
                /* d * sc * q, two f32 multiplies left to right */
                y[l] = d * (float)(int8_t)blk[sc + is] * (float)q1;
                y[l + 32] = d * (float)(int8_t)blk[sc + is + 2] * (float)q2;
                y[l + 64] = d * (float)(int8_t)blk[sc + is + 4] * (float)q3;
                y[l + 96] = d * (float)(int8_t)blk[sc + is + 6] * (float)q4;
            }
        }
    }
}

/* crates/llamd-quant/src/lib.rs:116-149. 0 ok; -1 unknown type; -2 partial
 * block; -3 source too short. Writes n floats to out. */
int orc_dequantize(int ty, const uint8_t *src, int64_t src_len, int64_t n, float *out) {
    int64_t need = orc_bytes_for(ty, n);
    if (need < 0) return (int)need;
    if (src_len < need) return -3;
    switch (ty) {
    case ORC_F32: memcpy(out, src, (size_t)n * 4); break;
    case ORC_F16:
        for (int64_t i = 0; i < n; i++) out[i] = orc_f16_to_f32(rd_u16(src + 2 * i));
        break;
    case ORC_Q8_0: dequantize_q8_0(src, n, out); break;
    case ORC_Q6K: dequantize_q6_k(src, n, out); break;
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* Q8_K quantizer and the integer dot                                        */
/* ------------------------------------------------------------------------ */

/* crates/llamd-quant/src/dot.rs:74-86: round half to even. */
int orc_nearest_int(float v) { return (int)nearbyintf(v); }

/* crates/llamd-quant/src/dot.rs:88-128. Blocks are returned as three planes:
 * qs[nblocks*256], d[nblocks], bsums[nblocks*16] (the split the reference's
 * own device FFI uses, crates/llamd-rocm/src/lib.rs:120-126). */
void orc_quantize_q8k(const float *x, int nblocks, int8_t *qs, float *d, int16_t *bsums) {
    for (int b = 0; b < nblocks; b++) {
        const float *chunk = x + (size_t)b * QK_K;
        int8_t *q = qs + (size_t)b * QK_K;
        int16_t *bs = bsums ? bsums + (size_t)b * (QK_K / 16) : NULL;
        float amax = 0.0f, max = 0.0f;
        for (int i = 0; i < QK_K; i++) {
            float a = fabsf(chunk[i]);
            if (a > amax) {
                amax = a;
                max = chunk[i];
            }
        }
        if (amax == 0.0f) {
            memset(q, 0, QK_K);
            if (bs) memset(bs, 0, sizeof(int16_t) * (QK_K / 16));
            d[b] = 0.0f;
            continue;
        }
        float iscale = -127.0f / max;
        for (int i = 0; i < QK_K; i++) {
            int v = orc_nearest_int(iscale * chunk[i]);
            if (v > 127) v = 127;
            q[i] = (int8_t)v;
        }
        if (bs) {
            for (int g = 0; g < QK_K / 16; g++) {
                int16_t s = 0;
                for (int i = 0; i < 16; i++) s = (int16_t)(s + q[g * 16 + i]);
                bs[g] = s;
            }
        }
        d[b] = 1.0f / iscale;
    }
}

/* crates/llamd-quant/src/dot.rs:138-196 */
float orc_dot_q6k_q8k(const uint8_t *w, const int8_t *aqs, const float *ad, int n) {
    const int QL = 0, QH = QK_K / 2, SC = QK_K / 2 + QK_K / 4, D = QK_K / 2 + QK_K / 4 + QK_K / 16;
    int nb = n / QK_K;
    float sums[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int i = 0; i < nb; i++) {
        const uint8_t *blk = w + (size_t)i * Q6K_BLOCK_BYTES;
        const int8_t *yq = aqs + (size_t)i * QK_K;
        int8_t aux8[QK_K];
        for (int half = 0; half < 2; half++) {
            int ql = QL + half * 64, qh = QH + half * 32, o = half * 128;
            for (int l = 0; l < 32; l++) {
                uint8_t h = blk[qh + l], lo0 = blk[ql + l], lo1 = blk[ql + l + 32];
                aux8[o + l] = (int8_t)((lo0 & 0x0F) | ((h & 3) << 4)) - 32;
                aux8[o + l + 32] = (int8_t)((lo1 & 0x0F) | (((h >> 2) & 3) << 4)) - 32;
                aux8[o + l + 64] = (int8_t)((lo0 >> 4) | (((h >> 4) & 3) << 4)) - 32;
                aux8[o + l + 96] = (int8_t)((lo1 >> 4) | (((h >> 6) & 3) << 4)) - 32;
            }
        }
        int32_t aux32[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int j = 0; j < QK_K / 16; j++) {
            int32_t scale = (int8_t)blk[SC + j];
            for (int half = 0; half < 2; half++) {
                int o = j * 16 + half * 8;
                for (int l = 0; l < 8; l++) {
                    int16_t p = (int16_t)((int16_t)yq[o + l] * (int16_t)aux8[o + l]);
                    aux32[l] += scale * (int32_t)p;
                }
            }
        }
        float d = orc_f16_to_f32(rd_u16(blk + D)) * ad[i];
        for (int l = 0; l < 8; l++) sums[l] += d * (float)aux32[l];
    }
    /* `sums.iter().sum()`: Rust's f32 Sum folds left to right from -0.0. */
    float total = -0.0f;
    for (int l = 0; l < 8; l++) total = total + sums[l];
    return total;
}

/* crates/llamd-quant/src/dot.rs:379-423: byte permutation into four planes. */
int orc_repack_q6k_planar(const uint8_t *src, int64_t src_len, int64_t rows, int64_t blocks,
                          uint8_t *out, int64_t off[5]) {
    int64_t n = rows * blocks;
    if (src_len < n * Q6K_BLOCK_BYTES) return -1;
    int64_t ql = 0, qh = ql + n * 128, sc = qh + n * 64, d = sc + n * 16;
    off[0] = ql; off[1] = qh; off[2] = sc; off[3] = d; off[4] = d + n * 2;
    if (!out) return 0;
    for (int64_t i = 0; i < n; i++) {
        const uint8_t *b = src + i * Q6K_BLOCK_BYTES;
        memcpy(out + ql + i * 128, b, 128);
        memcpy(out + qh + i * 64, b + 128, 64);
        memcpy(out + sc + i * 16, b + 192, 16);
        memcpy(out + d + i * 2, b + 208, 2);
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* a small row-parallel helper. Rows are independent, so splitting them over  */
/* threads changes no result.                                                */
/* ------------------------------------------------------------------------ */

typedef void (*row_fn)(int64_t r0, int64_t r1, void *ctx);

/* A persistent pool: workers are started once and parked between calls (a short
 * spin, then a condition variable), so that a call costs a few microseconds
 * instead of a thread creation per worker. A decode token makes ~1500 such
 * calls. Chunks of rows are handed out through an atomic counter; the calling
 * thread works too. One call at a time (callers are serialised by pool.call). */
#define ORC_MAX_THREADS 256
static struct {
    pthread_mutex_t call, mu;
    pthread_cond_t cv;
    pthread_t th[ORC_MAX_THREADS];
    int n_workers, sleepers, atfork_set;
    unsigned gen;                 /* bumped once per call (atomic) */
    int use;                      /* workers with id < use take chunks */
    int active;                   /* workers that have not yet finished the current call (atomic) */
    row_fn fn;
    void *ctx;
    int64_t rows, chunk, next;    /* next: atomic */
} pool = {PTHREAD_MUTEX_INITIALIZER, PTHREAD_MUTEX_INITIALIZER, PTHREAD_COND_INITIALIZER, {0}, 0, 0, 0, 0, 0, 0, NULL, NULL, 0, 0, 0};

static void pool_take_chunks(void) {
    for (;;) {
        int64_t r0 = __atomic_fetch_add(&pool.next, pool.chunk, __ATOMIC_RELAXED);
        if (r0 >= pool.rows) return;
        int64_t r1 = r0 + pool.chunk > pool.rows ? pool.rows : r0 + pool.chunk;
        pool.fn(r0, r1, pool.ctx);
    }
}
static void *pool_worker(void *arg) {
    int id = (int)(intptr_t)arg;
    unsigned seen = 0;
    for (;;) {
        int spins = 0;
        while (__atomic_load_n(&pool.gen, __ATOMIC_ACQUIRE) == seen) {
            if (++spins < 4000) {
#if defined(__x86_64__) || defined(__i386__)
                __builtin_ia32_pause();
#endif
                continue;
            }
            pthread_mutex_lock(&pool.mu);
            pool.sleepers++;
            while (__atomic_load_n(&pool.gen, __ATOMIC_ACQUIRE) == seen) pthread_cond_wait(&pool.cv, &pool.mu);
            pool.sleepers--;
            pthread_mutex_unlock(&pool.mu);
        }
        seen = __atomic_load_n(&pool.gen, __ATOMIC_ACQUIRE);
        if (id < pool.use) pool_take_chunks();
        __atomic_fetch_sub(&pool.active, 1, __ATOMIC_RELEASE);
    }
    return NULL;
}
/* a forked child has none of the parent's threads */
static void pool_after_fork(void) {
    pool.n_workers = 0;
    pool.sleepers = 0;
    pthread_mutex_init(&pool.call, NULL);
    pthread_mutex_init(&pool.mu, NULL);
    pthread_cond_init(&pool.cv, NULL);
}
static void parallel_rows(int64_t rows, int threads, row_fn fn, void *ctx) {
    if (threads <= 1 || rows < 2 * threads) {
        fn(0, rows, ctx);
        return;
    }
    if (threads > ORC_MAX_THREADS) threads = ORC_MAX_THREADS;
    pthread_mutex_lock(&pool.call);
    if (!pool.atfork_set) {
        pthread_atfork(NULL, NULL, pool_after_fork);
        pool.atfork_set = 1;
    }
    while (pool.n_workers < threads - 1) {
        if (pthread_create(&pool.th[pool.n_workers], NULL, pool_worker, (void *)(intptr_t)pool.n_workers) != 0) break;
        pthread_detach(pool.th[pool.n_workers]);
        pool.n_workers++;
    }
    pool.fn = fn;
    pool.ctx = ctx;
    pool.rows = rows;
    pool.chunk = rows / (4 * (int64_t)threads);
    if (pool.chunk < 1) pool.chunk = 1;
    pool.use = threads - 1;
    __atomic_store_n(&pool.next, 0, __ATOMIC_RELAXED);
    __atomic_store_n(&pool.active, pool.n_workers, __ATOMIC_RELAXED);
    __atomic_fetch_add(&pool.gen, 1, __ATOMIC_RELEASE);
    pthread_mutex_lock(&pool.mu);
    if (pool.sleepers) pthread_cond_broadcast(&pool.cv);
    pthread_mutex_unlock(&pool.mu);
    pool_take_chunks();
    while (__atomic_load_n(&pool.active, __ATOMIC_ACQUIRE) != 0) {
#if defined(__x86_64__) || defined(__i386__)
        __builtin_ia32_pause();
#endif
    }
    pthread_mutex_unlock(&pool.call);
}

/* ------------------------------------------------------------------------ */
/* Model::matvec_quant and friends                                           */
/* ------------------------------------------------------------------------ */

typedef struct {
    const uint8_t *w; const int8_t *qs; const float *d; int k; float *y;
} mvq_ctx;
static void mvq_rows(int64_t r0, int64_t r1, void *p) {
    mvq_ctx *c = (mvq_ctx *)p;
    size_t row_bytes = (size_t)(c->k / QK_K) * Q6K_BLOCK_BYTES;
    for (int64_t r = r0; r < r1; r++) c->y[r] = orc_dot_q6k_q8k(c->w + r * row_bytes, c->qs, c->d, c->k);
}

/* Q6_K rows against an already quantized activation: the loop at
 * crates/llamd-models/src/model.rs:268-275 (and :309-317 for one expert). */
void orc_matvec_q6k_q8k(const uint8_t *w, const int8_t *qs, const float *d, int k, int64_t rows,
                        float *y, int threads) {
    mvq_ctx c = {w, qs, d, k, y};
    parallel_rows(rows, threads, mvq_rows, &c);
}

/* crates/llamd-models/src/model.rs:265-275: quantize x once, dot every row. */
int orc_matvec_q6k(const uint8_t *w, const float *x, int k, int64_t rows, float *y, int threads) {
    if (k <= 0 || k % QK_K) return -2;
    int nb = k / QK_K;
    int8_t *qs = (int8_t *)malloc((size_t)k);
    float *d = (float *)malloc(sizeof(float) * nb);
    orc_quantize_q8k(x, nb, qs, d, NULL);
    orc_matvec_q6k_q8k(w, qs, d, k, rows, y, threads);
    free(qs);
    free(d);
    return 0;
}

typedef struct { const float *w; const float *x; int k; float *y; } mvf_ctx;
static void mvf_rows(int64_t r0, int64_t r1, void *p) {
    mvf_ctx *c = (mvf_ctx *)p;
    for (int64_t r = r0; r < r1; r++) {
        const float *row = c->w + r * c->k;
        /* row.iter().zip(x).map(|(a,b)| a*b).sum() */
        float acc = -0.0f;
        for (int t = 0; t < c->k; t++) acc = acc + row[t] * c->x[t];
        c->y[r] = acc;
    }
}

/* crates/llamd-models/src/model.rs:253-263: any type without a quantized
 * kernel (F32, F16, Q8_0) is dequantized whole, then dotted in f32 in order. */
int orc_matvec_dequant(int ty, const uint8_t *w, const float *x, int k, int64_t rows, float *y,
                       int threads) {
    int64_t n = (int64_t)k * rows;
    int64_t need = orc_bytes_for(ty, n);
    if (need < 0) return (int)need;
    const float *wf;
    float *tmp = NULL;
    if (ty == ORC_F32) {
        wf = (const float *)w;
    } else {
        tmp = (float *)malloc(sizeof(float) * (size_t)n);
        orc_dequantize(ty, w, need, n, tmp);
        wf = tmp;
    }
    mvf_ctx c = {wf, x, k, y};
    parallel_rows(rows, threads, mvf_rows, &c);
    free(tmp);
    return 0;
}

/* ------------------------------------------------------------------------ */
/* CpuBackend ops: crates/llamd-cpu/src/lib.rs                               */
/* ------------------------------------------------------------------------ */

/* :55-75. No learned weight folded in. */
void orc_rms_norm(const float *x, int n, int rows, float eps, float *out) {
    for (int r = 0; r < rows; r++) {
        const float *src = x + (size_t)r * n;
        float sum = 0.0f;
        for (int i = 0; i < n; i++) sum += src[i] * src[i];
        float scale = 1.0f / sqrtf(sum / (float)n + eps);
        for (int i = 0; i < n; i++) out[(size_t)r * n + i] = src[i] * scale;
    }
}

/* :81-101 */
void orc_softmax(const float *x, int n, int rows, float *out) {
    for (int r = 0; r < rows; r++) {
        const float *src = x + (size_t)r * n;
        float *dst = out + (size_t)r * n;
        float max = -INFINITY;
        for (int i = 0; i < n; i++) max = fmaxf(max, src[i]);
        float sum = 0.0f;
        for (int i = 0; i < n; i++) {
            float e = expf(src[i] - max);
            dst[i] = e;
            sum += e;
        }
        float inv = 1.0f / sum;
        for (int i = 0; i < n; i++) dst[i] *= inv;
    }
}

/* :103-106 */
void orc_silu(const float *x, int64_t n, float *out) {
    for (int64_t i = 0; i < n; i++) out[i] = x[i] / (1.0f + expf(-x[i]));
}
/* :108-118 */
void orc_add(const float *a, const float *b, int64_t n, float *out) {
    for (int64_t i = 0; i < n; i++) out[i] = a[i] + b[i];
}
void orc_mul(const float *a, const float *b, int64_t n, float *out) {
    for (int64_t i = 0; i < n; i++) out[i] = a[i] * b[i];
}
void orc_scale(const float *a, float by, int64_t n, float *out) {
    for (int64_t i = 0; i < n; i++) out[i] = a[i] * by;
}

/* :126-149. w [k,m], x [k,n] -> out [m,n], out[j*m+i]. */
void orc_matmul(const float *w, const float *x, int k, int m, int n, float *out) {
    for (int j = 0; j < n; j++) {
        const float *xr = x + (size_t)j * k;
        for (int i = 0; i < m; i++) {
            const float *wr = w + (size_t)i * k;
            float acc = 0.0f;
            for (int t = 0; t < k; t++) acc += wr[t] * xr[t];
            out[(size_t)j * m + i] = acc;
        }
    }
}

/* :158-209. NeoX pairing (i, i + d/2). */
int orc_rope(const float *x, int row_len, int rows, const uint32_t *positions, int head_dim,
             float freq_base, float freq_scale, float *out) {
    int d = head_dim;
    if (d % 2 != 0 || row_len % d != 0) return -2;
    int heads = row_len / d, half = d / 2;
    for (int r = 0; r < rows; r++) {
        float pos = (float)positions[r] * freq_scale;
        const float *src = x + (size_t)r * row_len;
        float *dst = out + (size_t)r * row_len;
        for (int h = 0; h < heads; h++) {
            int base = h * d;
            for (int i = 0; i < half; i++) {
                float exponent = 2.0f * (float)i / (float)d;
                float theta = pos / powf(freq_base, exponent);
                float s = sinf(theta), c = cosf(theta);
                float a = src[base + i], b = src[base + i + half];
                dst[base + i] = a * c - b * s;
                dst[base + i + half] = a * s + b * c;
            }
        }
    }
    return 0;
}

/* The sin/cos pair the rope above uses at (pos, i): lets a caller tabulate
 * the host libm's values. */
void orc_rope_angles(uint32_t pos, int head_dim, float freq_base, float freq_scale, float *sin_out,
                     float *cos_out) {
    float p = (float)pos * freq_scale;
    for (int i = 0; i < head_dim / 2; i++) {
        float exponent = 2.0f * (float)i / (float)head_dim;
        float theta = p / powf(freq_base, exponent);
        sin_out[i] = sinf(theta);
        cos_out[i] = cosf(theta);
    }
}

/* :211-224. -2 when an id is outside the table. */
int orc_get_rows(const float *table, int row_len, int rows, const uint32_t *ids, int n_ids,
                 float *out) {
    for (int i = 0; i < n_ids; i++) {
        if (ids[i] >= (uint32_t)rows) return -2;
        memcpy(out + (size_t)i * row_len, table + (size_t)ids[i] * row_len, sizeof(float) * row_len);
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* route: crates/llamd-models/src/moe.rs:50-113                              */
/* ------------------------------------------------------------------------ */

#define WEIGHT_SUM_FLOOR 6.103515625e-5f

int orc_route(const float *logits, int n, int n_used, int32_t *experts, float *weights_raw,
              float *weight_sum, float *weights, float *probs_out) {
    if (n_used == 0 || n_used > n) return -2;
    float *probs = (float *)malloc(sizeof(float) * n);
    int32_t *idx = (int32_t *)malloc(sizeof(int32_t) * n);
    float max = -INFINITY;
    for (int i = 0; i < n; i++) max = fmaxf(max, logits[i]);
    for (int i = 0; i < n; i++) probs[i] = expf(logits[i] - max);
    float total = -0.0f; /* probs.iter().sum() */
    for (int i = 0; i < n; i++) total = total + probs[i];
    for (int i = 0; i < n; i++) probs[i] /= total;
    /* Stable sort, probability descending then index ascending. An insertion
     * sort is stable and n is 128. NaN compares Equal in the reference
     * (partial_cmp().unwrap_or(Equal)) and then falls to the index. */
    for (int i = 0; i < n; i++) idx[i] = i;
    for (int i = 1; i < n; i++) {
        int32_t v = idx[i];
        int j = i - 1;
        while (j >= 0) {
            int32_t u = idx[j];
            /* does v sort strictly before u? */
            int before;
            if (probs[v] > probs[u]) before = 1;
            else if (probs[v] < probs[u]) before = 0;
            else before = v < u;
            if (!before) break;
            idx[j + 1] = u;
            j--;
        }
        idx[j + 1] = v;
    }
    float sum = -0.0f; /* weights_raw.iter().sum::<f32>() */
    for (int i = 0; i < n_used; i++) {
        experts[i] = idx[i];
        weights_raw[i] = probs[idx[i]];
        sum = sum + weights_raw[i];
    }
    sum = fmaxf(sum, WEIGHT_SUM_FLOOR);
    *weight_sum = sum;
    for (int i = 0; i < n_used; i++) weights[i] = weights_raw[i] / sum;
    if (probs_out) memcpy(probs_out, probs, sizeof(float) * n);
    free(probs);
    free(idx);
    return 0;
}

/* f32::exp as the reference's CPU ops call it (the host libm), elementwise: for checking the device's exponential. */
void orc_expf(const float *x, int64_t n, float *out) {
    for (int64_t i = 0; i < n; i++) out[i] = expf(x[i]);
}

/* ------------------------------------------------------------------------ */
/* attend: crates/llamd-runtime/src/attention.rs:62-125                      */
/* ------------------------------------------------------------------------ */

typedef struct {
    const float *q, *k, *v;
    int n_kv, n_head, n_head_kv, head_dim;
    float *out;
} attend_ctx;
/* heads [h0, h1): each head is computed exactly as the reference's loop body does */
static void attend_heads(int64_t h0, int64_t h1, void *p) {
    const attend_ctx *c = (const attend_ctx *)p;
    const float *q = c->q, *k = c->k, *v = c->v;
    float *out = c->out;
    int n_kv = c->n_kv, head_dim = c->head_dim;
    int kv_dim = c->n_head_kv * head_dim;
    float scale = 1.0f / sqrtf((float)head_dim);
    int ratio = c->n_head / c->n_head_kv;
    float *logits = (float *)malloc(sizeof(float) * n_kv);
    for (int h = (int)h0; h < (int)h1; h++) {
        int kvh = h / ratio, qo = h * head_dim;
        for (int d = 0; d < head_dim; d++) out[qo + d] = 0.0f;
        for (int t = 0; t < n_kv; t++) {
            size_t ko = (size_t)t * kv_dim + kvh * head_dim;
            float dot = 0.0f;
            for (int d = 0; d < head_dim; d++) dot += q[qo + d] * k[ko + d];
            logits[t] = dot * scale;
        }
        float max = -INFINITY;
        for (int t = 0; t < n_kv; t++) max = fmaxf(max, logits[t]);
        float sum = 0.0f;
        for (int t = 0; t < n_kv; t++) {
            logits[t] = expf(logits[t] - max);
            sum += logits[t];
        }
        float inv = 1.0f / sum;
        for (int t = 0; t < n_kv; t++) {
            float w = logits[t] * inv;
            size_t vo = (size_t)t * kv_dim + kvh * head_dim;
            for (int d = 0; d < head_dim; d++) out[qo + d] += w * v[vo + d];
        }
    }
    free(logits);
}

/* Heads are independent, so handing them to several threads changes no result. */
int orc_attend_mt(const float *q, const float *k, const float *v, int n_kv, int n_head, int n_head_kv,
                  int head_dim, float *out, int threads) {
    if (n_head_kv == 0 || n_head % n_head_kv != 0 || head_dim == 0 || n_kv == 0) return -2;
    attend_ctx c = {q, k, v, n_kv, n_head, n_head_kv, head_dim, out};
    if (threads > n_head / 2) threads = n_head / 2;
    parallel_rows(n_head, threads, attend_heads, &c);
    return 0;
}
int orc_attend(const float *q, const float *k, const float *v, int n_kv, int n_head, int n_head_kv,
               int head_dim, float *out) {
    return orc_attend_mt(q, k, v, n_kv, n_head, n_head_kv, head_dim, out, 1);
}

/* ------------------------------------------------------------------------ */
/* the decode loop: crates/llamd-runtime/src/layer.rs                        */
/* ------------------------------------------------------------------------ */

/* Where one expert's Q6_K bytes live. which: 0 gate, 1 up, 2 down. Lets a
 * caller keep 128 experts x 48 layers out of host memory and produce the
 * slice on demand; Model::expert (crates/llamd-models/src/model.rs:188-227)
 * is the same contiguous slice of the [k, rows, n_expert] tensor. */
typedef const uint8_t *(*orc_expert_fn)(void *user, int layer, int which, int expert);

typedef struct {
    int32_t n_layer, n_embd, n_head, n_head_kv, head_dim;
    int32_t n_expert, n_expert_used, n_ff_expert, n_vocab;
    float rope_freq_base, rms_eps;
    const uint8_t *tok_embd;       /* Q6_K [n_vocab rows x n_embd] */
    const float *output_norm;      /* [n_embd] */
    const uint8_t *output;         /* Q6_K [n_vocab rows x n_embd] */
    const float *const *attn_norm; /* per layer [n_embd] */
    const uint8_t *const *attn_q;  /* per layer Q6_K [n_head*hd x n_embd] */
    const uint8_t *const *attn_k;
    const uint8_t *const *attn_v;
    const float *const *attn_q_norm; /* per layer [hd] */
    const float *const *attn_k_norm;
    const uint8_t *const *attn_out;  /* Q6_K [n_embd x n_head*hd] */
    const float *const *ffn_norm;
    const float *const *ffn_gate_inp; /* F32 [n_expert x n_embd] */
    const uint8_t *const *ffn_gate_exps; /* Q6_K [n_expert][n_ff x n_embd], or NULL */
    const uint8_t *const *ffn_up_exps;
    const uint8_t *const *ffn_down_exps; /* Q6_K [n_expert][n_embd x n_ff] */
    orc_expert_fn expert_fn;             /* used when the arrays above are NULL */
    void *expert_user;
    int32_t threads;
} orc_model;

/* KvCache: crates/llamd-runtime/src/kv.rs:27-170, f32, [pos][kv_dim] per layer.
 * f16_store (no counterpart in the reference, whose caches are f32; the benchmark configuration names an f16 cache): a
 * value is rounded to IEEE binary16, nearest-even, when it is appended, and kept as the f32 that binary16 value widens
 * to. Everything downstream is the same arithmetic. */
typedef struct {
    int32_t n_layer, kv_dim, capacity;
    float **k;
    float **v;
    int32_t f16_store;
} orc_kv;

/* f32 -> binary16 (round to nearest, ties to even; overflow to infinity; subnormals kept) -> f32. */
static float round_to_f16(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    const uint32_t sign = u & 0x80000000u;
    uint32_t a = u & 0x7FFFFFFFu;
    if (a >= 0x7F800000u) return x; /* inf, NaN */
    if (a >= 0x477FF000u) {         /* rounds to 65536 or more: infinity */
        a = 0x7F800000u;
    } else if (a >= 0x38800000u) {  /* normal in binary16: keep 10 mantissa bits */
        const uint32_t lsb = (a >> 13) & 1u;
        a = (a + 0x0FFFu + lsb) & ~0x1FFFu;
    } else {                        /* subnormal in binary16 (or zero): multiples of 2^-24 */
        float f;
        memcpy(&f, &a, 4);
        f = nearbyintf(f * 16777216.0f) / 16777216.0f; /* exact: nearbyintf rounds ties to even under the default mode */
        memcpy(&a, &f, 4);
    }
    a |= sign;
    float r;
    memcpy(&r, &a, 4);
    return r;
}
void orc_kv_set_f16(orc_kv *kv, int on) { if (kv) kv->f16_store = on != 0; }
float orc_round_to_f16(float x) { return round_to_f16(x); }

orc_kv *orc_kv_new(int n_layer, int kv_dim, int capacity) {
    if (n_layer <= 0 || kv_dim <= 0 || capacity <= 0) return NULL;
    orc_kv *kv = (orc_kv *)calloc(1, sizeof(orc_kv));
    kv->n_layer = n_layer; kv->kv_dim = kv_dim; kv->capacity = capacity;
    kv->k = (float **)calloc(n_layer, sizeof(float *));
    kv->v = (float **)calloc(n_layer, sizeof(float *));
    for (int i = 0; i < n_layer; i++) {
        kv->k[i] = (float *)calloc((size_t)capacity * kv_dim, sizeof(float));
        kv->v[i] = (float *)calloc((size_t)capacity * kv_dim, sizeof(float));
    }
    return kv;
}
void orc_kv_free(orc_kv *kv) {
    if (!kv) return;
    for (int i = 0; i < kv->n_layer; i++) { free(kv->k[i]); free(kv->v[i]); }
    free(kv->k); free(kv->v); free(kv);
}
const float *orc_kv_keys(const orc_kv *kv, int layer) { return kv->k[layer]; }
const float *orc_kv_values(const orc_kv *kv, int layer) { return kv->v[layer]; }

/* layer.rs:62-79 */
static void per_head_rms_norm(const float *x, const float *w, int n_head, int hd, float eps, float *out) {
    orc_rms_norm(x, hd, n_head, eps, out);
    for (int h = 0; h < n_head; h++)
        for (int d = 0; d < hd; d++) out[h * hd + d] *= w[d];
}

static const uint8_t *expert_ptr(const orc_model *m, int il, int which, int e) {
    const uint8_t *const *arr = which == 0 ? m->ffn_gate_exps : which == 1 ? m->ffn_up_exps : m->ffn_down_exps;
    if (arr && arr[il]) {
        size_t per = (size_t)m->n_ff_expert * m->n_embd / QK_K * Q6K_BLOCK_BYTES;
        return arr[il] + (size_t)e * per;
    }
    return m->expert_fn(m->expert_user, il, which, e);
}

/* Optional per-layer intermediates, named as LayerTrace (layer.rs:39-57). Any
 * pointer may be NULL. */
typedef struct {
    float *attn_norm, *q, *k, *v, *q_roped, *k_roped, *attn_out, *kqv_out, *ffn_inp, *ffn_norm;
    float *moe_logits, *moe_probs;
    int32_t *experts;
    float *weights;
    float *ffn_out;
    float *x_out;
} orc_trace;

#define CPY(dst, src, n) do { if (dst) memcpy(dst, src, sizeof(float) * (n)); } while (0)

/* forward_layer (layer.rs:85-203) + moe_ffn (:230-260) + the residual at
 * :281-287, for one token. x is updated in place. */
static int forward_one_layer(const orc_model *m, int il, float *x, uint32_t pos, orc_kv *kv, orc_trace *tr) {
    int n_embd = m->n_embd, n_head = m->n_head, n_head_kv = m->n_head_kv, hd = m->head_dim;
    int kv_dim = n_head_kv * hd, qd = n_head * hd, th = m->threads;
    int n_ffe = m->n_ff_expert, n_used = m->n_expert_used;
    if ((int)pos >= kv->capacity) return -2;
    size_t nf = (size_t)n_embd * 6 + (size_t)qd * 4 + (size_t)kv_dim * 5 + (size_t)m->n_expert * 2 +
                (size_t)n_ffe * 3 + 64;
    float *buf = (float *)malloc(sizeof(float) * nf), *p = buf;
    float *norm = p; p += n_embd;
    float *attn_norm = p; p += n_embd;
    float *q = p; p += qd;
    float *k = p; p += kv_dim;
    float *v = p; p += kv_dim;
    float *qn = p; p += qd;
    float *kn = p; p += kv_dim;
    float *qr = p; p += qd;
    float *kr = p; p += kv_dim;
    float *attn = p; p += qd;
    float *kqv = p; p += n_embd;
    float *ffn_inp = p; p += n_embd;
    float *ffn_norm = p; p += n_embd;
    float *logits = p; p += m->n_expert;
    float *probs = p; p += m->n_expert;
    float *gate = p; p += n_ffe;
    float *up = p; p += n_ffe;
    float *act = p; p += n_ffe;
    float *down = p; p += n_embd;
    float *w8 = p; p += 8 + 8 + 8; (void)p;
    int32_t experts[64];
    float wraw[64], wsum;
    float *weights = w8;
    if (n_used > 64) { free(buf); return -2; }

    orc_rms_norm(x, n_embd, 1, m->rms_eps, norm);
    orc_mul(norm, m->attn_norm[il], n_embd, attn_norm);
    orc_matvec_q6k(m->attn_q[il], attn_norm, n_embd, qd, q, th);
    orc_matvec_q6k(m->attn_k[il], attn_norm, n_embd, kv_dim, k, th);
    orc_matvec_q6k(m->attn_v[il], attn_norm, n_embd, kv_dim, v, th);
    if (m->attn_q_norm && m->attn_q_norm[il]) per_head_rms_norm(q, m->attn_q_norm[il], n_head, hd, m->rms_eps, qn);
    else memcpy(qn, q, sizeof(float) * qd);
    if (m->attn_k_norm && m->attn_k_norm[il]) per_head_rms_norm(k, m->attn_k_norm[il], n_head_kv, hd, m->rms_eps, kn);
    else memcpy(kn, k, sizeof(float) * kv_dim);
    orc_rope(qn, qd, 1, &pos, hd, m->rope_freq_base, 1.0f, qr);
    orc_rope(kn, kv_dim, 1, &pos, hd, m->rope_freq_base, 1.0f, kr);
    memcpy(kv->k[il] + (size_t)pos * kv_dim, kr, sizeof(float) * kv_dim);
    memcpy(kv->v[il] + (size_t)pos * kv_dim, v, sizeof(float) * kv_dim);
    if (kv->f16_store) {
        float *kd = kv->k[il] + (size_t)pos * kv_dim, *vd = kv->v[il] + (size_t)pos * kv_dim;
        for (int i = 0; i < kv_dim; i++) {
            kd[i] = round_to_f16(kd[i]);
            vd[i] = round_to_f16(vd[i]);
        }
    }
    int n_kv = (int)pos + 1;
    orc_attend_mt(qr, kv->k[il], kv->v[il], n_kv, n_head, n_head_kv, hd, attn, th);
    orc_matvec_q6k(m->attn_out[il], attn, qd, n_embd, kqv, th);
    orc_add(x, kqv, n_embd, ffn_inp);
    orc_rms_norm(ffn_inp, n_embd, 1, m->rms_eps, norm);
    orc_mul(norm, m->ffn_norm[il], n_embd, ffn_norm);
    orc_matvec_dequant(ORC_F32, (const uint8_t *)m->ffn_gate_inp[il], ffn_norm, n_embd, m->n_expert, logits, th);
    orc_softmax(logits, m->n_expert, 1, probs);
    int rc = orc_route(logits, m->n_expert, n_used, experts, wraw, &wsum, weights, NULL);
    if (rc) { free(buf); return rc; }

    /* moe_ffn */
    float *out = norm; /* reuse */
    for (int i = 0; i < n_embd; i++) out[i] = 0.0f;
    for (int s = 0; s < n_used; s++) {
        int e = experts[s];
        float w = weights[s];
        orc_matvec_q6k(expert_ptr(m, il, 0, e), ffn_norm, n_embd, n_ffe, gate, th);
        orc_matvec_q6k(expert_ptr(m, il, 1, e), ffn_norm, n_embd, n_ffe, up, th);
        orc_silu(gate, n_ffe, act);
        orc_mul(act, up, n_ffe, act);
        orc_matvec_q6k(expert_ptr(m, il, 2, e), act, n_ffe, n_embd, down, th);
        for (int i = 0; i < n_embd; i++) out[i] += w * down[i];
    }
    if (tr) {
        CPY(tr->attn_norm, attn_norm, n_embd); CPY(tr->q, q, qd); CPY(tr->k, k, kv_dim); CPY(tr->v, v, kv_dim);
        CPY(tr->q_roped, qr, qd); CPY(tr->k_roped, kr, kv_dim); CPY(tr->attn_out, attn, qd);
        CPY(tr->kqv_out, kqv, n_embd); CPY(tr->ffn_inp, ffn_inp, n_embd); CPY(tr->ffn_norm, ffn_norm, n_embd);
        CPY(tr->moe_logits, logits, m->n_expert); CPY(tr->moe_probs, probs, m->n_expert);
        if (tr->experts) memcpy(tr->experts, experts, sizeof(int32_t) * n_used);
        CPY(tr->weights, weights, n_used); CPY(tr->ffn_out, out, n_embd);
    }
    /* x = ffn_inp; x += ffn (layer.rs:281-287) */
    for (int i = 0; i < n_embd; i++) x[i] = ffn_inp[i];
    for (int i = 0; i < n_embd; i++) x[i] += out[i];
    if (tr) CPY(tr->x_out, x, n_embd);
    free(buf);
    return 0;
}

/* One layer alone, for layer-level parity tests. */
int orc_forward_layer(const orc_model *m, int il, float *x, uint32_t pos, orc_kv *kv, orc_trace *tr) {
    return forward_one_layer(m, il, x, pos, kv, tr);
}

/* moe_ffn alone (layer.rs:230-260), given a routing. */
int orc_moe_ffn(const orc_model *m, int il, const float *x, const int32_t *experts, const float *weights,
                int n_used, float *out) {
    int n_embd = m->n_embd, n_ffe = m->n_ff_expert, th = m->threads;
    float *gate = (float *)malloc(sizeof(float) * (3 * (size_t)n_ffe + n_embd));
    float *up = gate + n_ffe, *act = up + n_ffe, *down = act + n_ffe;
    for (int i = 0; i < n_embd; i++) out[i] = 0.0f;
    for (int s = 0; s < n_used; s++) {
        int e = experts[s];
        if (e < 0 || e >= m->n_expert) { free(gate); return -2; }
        orc_matvec_q6k(expert_ptr(m, il, 0, e), x, n_embd, n_ffe, gate, th);
        orc_matvec_q6k(expert_ptr(m, il, 1, e), x, n_embd, n_ffe, up, th);
        orc_silu(gate, n_ffe, act);
        orc_mul(act, up, n_ffe, act);
        orc_matvec_q6k(expert_ptr(m, il, 2, e), act, n_ffe, n_embd, down, th);
        for (int i = 0; i < n_embd; i++) out[i] += weights[s] * down[i];
    }
    free(gate);
    return 0;
}

/* forward (layer.rs:268-304): embed, every layer, final norm, output
 * projection. The reference dequantizes the whole embedding table and takes
 * one row; dequantizing that row alone yields the same values. */
int orc_forward(const orc_model *m, uint32_t token, uint32_t pos, orc_kv *kv, float *logits,
                float *x_final /* nullable */) {
    if ((int)token >= m->n_vocab) return -2;
    int n_embd = m->n_embd;
    float *x = (float *)malloc(sizeof(float) * 2 * (size_t)n_embd);
    float *normed = x + n_embd;
    size_t row_bytes = (size_t)n_embd / QK_K * Q6K_BLOCK_BYTES;
    dequantize_q6_k(m->tok_embd + (size_t)token * row_bytes, n_embd, x);
    for (int il = 0; il < m->n_layer; il++) {
        int rc = forward_one_layer(m, il, x, pos, kv, NULL);
        if (rc) { free(x); return rc; }
    }
    orc_rms_norm(x, n_embd, 1, m->rms_eps, normed);
    orc_mul(normed, m->output_norm, n_embd, normed);
    if (x_final) memcpy(x_final, normed, sizeof(float) * n_embd);
    orc_matvec_q6k(m->output ? m->output : m->tok_embd, normed, n_embd, m->n_vocab, logits, m->threads);
    free(x);
    return 0;
}

/* Greedy pick, lowest index on an exact tie: what every device argmax in the
 * reference does (crates/llamd-rocm/kernels/llamd_forward.hip:368-372). */
int32_t orc_argmax(const float *x, int64_t n) {
    int64_t best = 0;
    for (int64_t i = 1; i < n; i++)
        if (x[i] > x[best]) best = i;
    return (int32_t)best;
}
