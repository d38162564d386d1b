/*
 * CPU oracle for the paged KV-cache decode path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference's own CPU
 * implementation of the path (qubivex, a Rust workspace).  It is the checker the
 * CUDA kernels are compared against and the CPU baseline that is timed beside
 * them.  Nothing in the shipped library links, loads or calls it.
 *
 * Every function cites the reference file:line it follows (paths are relative to the
 * reference project's root).  Where the reference has no counterpart (reduced
 * precision KV, block sizes other than 256, the position-major "native" layout,
 * block copies for copy-on-write and compaction) the function says so: for those
 * the restatement is the only authority and their parity is unpinned by any
 * reference test.
 *
 * Pinned against the reference's own known-answer tests (see tests/test_oracle_pins.py):
 *   crates/qubivex-compute/src/math.rs:196-228   exp edges and the 2-ulp sweep
 *   crates/qubivex-arch/src/ops.rs:301-319       attention of one position, softmax sum
 *   crates/qubivex-compute/src/reduce.rs:53-73   64-lane dot against f64
 *   crates/qubivex-compute/src/discrete.rs:247-329 the pool's address identities
 *
 * Build: gcc -O3 -ffp-contract=off (no value-changing optimisation); fmaf() is used
 * exactly where the reference uses f32::mul_add.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ---- status codes, the same numbers the CUDA library returns ------------------ */
#define QVO_OK 0
#define QVO_ERR_SHAPE (-1)
#define QVO_ERR_UNSUPPORTED (-2)

/* ---- element types and layouts -------------------------------------------------- */
enum { QVO_F32 = 0, QVO_BF16 = 1, QVO_F16 = 2 };
enum { QVO_LAYOUT_REFERENCE = 0, QVO_LAYOUT_NATIVE = 1 };

typedef struct {
    uint32_t block_tokens; /* positions per block (the reference's KV_BLOCK is 256) */
    uint32_t kv_heads;
    uint32_t head_dim;
    uint32_t dtype;  /* QVO_F32 / QVO_BF16 / QVO_F16 */
    uint32_t layout; /* QVO_LAYOUT_* */
} qvo_geometry;

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* ================================================================================
 * math.rs
 * ============================================================================== */

/* crates/qubivex-compute/src/math.rs:13-35 — the constants, as bit patterns. */
#define LOG2E_BITS 0x3fb8aa3bu /* std::f32::consts::LOG2_E */
#define LN2_HI_BITS 0x3f317200u
#define LN2_LO_BITS 0x35bfbe8eu
static const uint32_t EXP_P[6] = {0x39506967u, 0x3ab743ceu, 0x3c088908u,
                                  0x3d2aa9c1u, 0x3e2aaaaau, 0x3f000000u};

/* crates/qubivex-compute/src/math.rs:39-42 */
static inline float pow2i(int k) { return u2f((uint32_t)(k + 127) << 23); }

/* crates/qubivex-compute/src/math.rs:50-75 — portable exp, fixed bits everywhere. */
float qvo_exp(float x) {
    if (x != x) return x;
    if (x > 88.72284f) return INFINITY;
    if (x < -87.33655f) return 0.0f;
    const float shift = 12582912.0f;
    float kf = (x * u2f(LOG2E_BITS) + shift) - shift; /* -ffp-contract=off: never fused */
    float r = fmaf(-kf, u2f(LN2_HI_BITS), x);
    r = fmaf(-kf, u2f(LN2_LO_BITS), r);
    float p = u2f(EXP_P[0]);
    for (int c = 1; c < 6; c++) p = fmaf(p, r, u2f(EXP_P[c]));
    float y = fmaf(p, r * r, r) + 1.0f;
    int k = (int)kf;
    int k1 = k >> 1;
    float v = (y * pow2i(k1)) * pow2i(k - k1);
    return v < 1.17549435e-38f ? 0.0f : v;
}

/* The same over an array (test support: the 2-ulp sweep visits millions of points). */
void qvo_exp_array(const float *x, float *y, size_t n) {
    for (size_t i = 0; i < n; i++) y[i] = qvo_exp(x[i]);
}

/* Rust's f32::max: the non-NaN operand when one is NaN. */
static inline float max_rust(float a, float b) {
    if (a != a) return b;
    if (b != b) return a;
    return a > b ? a : b;
}

/* crates/qubivex-compute/src/math.rs:120-130 — max-subtracted, sequential sum. */
void qvo_softmax(float *x, size_t n) {
    float m = -INFINITY;
    for (size_t j = 0; j < n; j++) m = max_rust(m, x[j]);
    float sum = 0.0f;
    for (size_t j = 0; j < n; j++) {
        x[j] = qvo_exp(x[j] - m);
        sum += x[j];
    }
    for (size_t j = 0; j < n; j++) x[j] /= sum;
}

/* crates/qubivex-compute/src/math.rs:134-136 — left fold of fused multiply-adds. */
static inline float dot_seq(const float *a, const float *b, size_t d) {
    float s = 0.0f;
    for (size_t i = 0; i < d; i++) s = fmaf(a[i], b[i], s);
    return s;
}

/* crates/qubivex-compute/src/math.rs:142-155 — causal attention of one query head over
 * positions 0..=pos of one KV head; k and v hold d values per position. */
void qvo_attend(const float *q, const float *k, const float *v, size_t d, size_t pos,
                float *out, float *scores) {
    float scale = 1.0f / sqrtf((float)d);
    for (size_t t = 0; t <= pos; t++) scores[t] = dot_seq(q, k + t * d, d) * scale;
    qvo_softmax(scores, pos + 1);
    for (size_t i = 0; i < d; i++) out[i] = 0.0f;
    for (size_t t = 0; t <= pos; t++) {
        float p = scores[t];
        const float *vr = v + t * d;
        for (size_t i = 0; i < d; i++) out[i] = fmaf(p, vr[i], out[i]);
    }
}

/* crates/qubivex-compute/src/reduce.rs:12-47 — 64 lanes, fixed halving tree. */
float qvo_reduce_dot(const float *w, const float *x, size_t n) {
    float acc[64];
    for (int l = 0; l < 64; l++) acc[l] = 0.0f;
    size_t full = n / 64 * 64;
    for (size_t c = 0; c < full; c += 64)
        for (int l = 0; l < 64; l++) acc[l] = fmaf(w[c + l], x[c + l], acc[l]);
    for (size_t l = 0; full + l < n; l++) acc[l] = fmaf(w[full + l], x[full + l], acc[l]);
    for (int wd = 32; wd >= 4; wd /= 2)
        for (int i = 0; i < wd; i++) acc[i] += acc[i + wd];
    return (acc[0] + acc[1]) + (acc[2] + acc[3]);
}

/* crates/qubivex-compute/src/math.rs:115-117 */
float qvo_rms_scale_of(float ss, float n, float eps) { return 1.0f / sqrtf(ss / n + eps); }

/* crates/qubivex-compute/src/math.rs:92-108 */
void qvo_rms_norm(float *x, const float *w, size_t n, double eps) {
    float r = qvo_rms_scale_of(qvo_reduce_dot(x, x, n), (float)n, (float)eps);
    for (size_t i = 0; i < n; i++) x[i] = (x[i] * r) * w[i];
}

/* crates/qubivex-compute/src/math.rs:159-168 — NeoX pairs (i, i + d/2); cs = [cos.., sin..]. */
void qvo_rope_rotate(float *head, const float *cs, size_t d) {
    size_t half = d / 2;
    const float *c = cs, *s = cs + half;
    for (size_t i = 0; i < half; i++) {
        float x1 = head[i], x2 = head[i + half];
        head[i] = x1 * c[i] - x2 * s[i];
        head[i + half] = x2 * c[i] + x1 * s[i];
    }
}

/* crates/qubivex-backend-cpu/src/sim.rs:333-357 — what SimDevice::attention does to the raw
 * projections: clamp(-c, c) on q, k and v (Rust's clamp: a NaN stays, -0 stays), the full-width
 * norms of each token's q row and k row, RoPE on every head of q and k from the token's row. */
static float clamp_rust(float z, float c) { return z < -c ? -c : (z > c ? c : z); }
void qvo_attn_prelude(float *q, float *k_new, float *v_new, size_t s, size_t heads, size_t kvh, size_t d, int has_clip,
                      float clip, const float *q_norm, const float *k_norm, double eps, const float *rope) {
    size_t q_out = heads * d, kv_out = kvh * d;
    if (has_clip) {
        for (size_t i = 0; i < s * q_out; i++) q[i] = clamp_rust(q[i], clip);
        for (size_t i = 0; i < s * kv_out; i++) k_new[i] = clamp_rust(k_new[i], clip);
        for (size_t i = 0; i < s * kv_out; i++) v_new[i] = clamp_rust(v_new[i], clip);
    }
    if (q_norm && k_norm) {
        for (size_t t = 0; t < s; t++) qvo_rms_norm(q + t * q_out, q_norm, q_out, eps);
        for (size_t t = 0; t < s; t++) qvo_rms_norm(k_new + t * kv_out, k_norm, kv_out, eps);
    }
    for (size_t t = 0; t < s; t++) {
        const float *cs = rope + t * d;
        for (size_t h = 0; h < heads; h++) qvo_rope_rotate(q + t * q_out + h * d, cs, d);
        for (size_t h = 0; h < kvh; h++) qvo_rope_rotate(k_new + t * kv_out + h * d, cs, d);
    }
}

/* ================================================================================
 * Element conversion.  Widening bf16 is the reference's `bits << 16`
 * (crates/qubivex-backend-cpu/src/formats.rs:76-80).  Narrowing has no reference
 * counterpart: round to nearest even; a NaN keeps its sign and becomes quiet.
 * ============================================================================== */
uint16_t qvo_f32_to_bf16(float f) {
    uint32_t u = f2u(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
float qvo_bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }
void qvo_narrow_array(const float *x, uint16_t *y, size_t n, uint32_t dtype);

/* IEEE binary16, round to nearest even, NaN quiet with sign (no reference counterpart). */
uint16_t qvo_f32_to_f16(float f) {
    uint32_t u = f2u(f);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u | ((a >> 13) & 0x1ffu));
    if (a >= 0x47800000u) return (uint16_t)(sign | 0x7c00u); /* >= 65536: inf (65520.. rounds below) */
    if (a >= 0x38800000u) { /* normal half */
        uint32_t m = a - 0x38000000u; /* rebias 127 -> 15 */
        uint32_t r = m + 0xfffu + ((m >> 13) & 1u);
        return (uint16_t)(sign | (r >> 13)); /* a carry into the exponent is right, incl. -> inf */
    }
    if (a < 0x33000000u) return (uint16_t)sign; /* below half the smallest subnormal */
    /* subnormal half: value = mant * 2^(e-150), target unit 2^-24 */
    uint32_t e = a >> 23;
    uint32_t mant = (a & 0x7fffffu) | 0x800000u;
    uint32_t shift = 126u - e; /* 14..24 */
    uint32_t q = mant >> shift;
    uint32_t rem = mant & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1u);
    if (rem > half || (rem == half && (q & 1u))) q++;
    return (uint16_t)(sign | q);
}
float qvo_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
    if (e == 0x1fu) return u2f(sign | 0x7f800000u | (m << 13));
    if (e != 0) return u2f(sign | ((e + 112u) << 23) | (m << 13));
    if (m == 0) return u2f(sign);
    float v = (float)m * 5.9604644775390625e-8f; /* m * 2^-24, exact */
    return sign ? -v : v;
}

void qvo_narrow_array(const float *x, uint16_t *y, size_t n, uint32_t dtype) {
    for (size_t i = 0; i < n; i++) y[i] = dtype == QVO_BF16 ? qvo_f32_to_bf16(x[i]) : qvo_f32_to_f16(x[i]);
}
void qvo_widen_array(const uint16_t *x, float *y, size_t n, uint32_t dtype) {
    for (size_t i = 0; i < n; i++) y[i] = dtype == QVO_BF16 ? qvo_bf16_to_f32(x[i]) : qvo_f16_to_f32(x[i]);
}

/* ================================================================================
 * Pool layout.
 *
 * REFERENCE layout: crates/qubivex-compute/src/discrete.rs:247-329, with the constant
 * KV_BLOCK = 256 generalised to `block_tokens` and the f32 word generalised to one
 * element: a block holds the keys dimension-major [kv_head][d][B], then the values
 * position-major [B][kv_head][d].
 *
 * NATIVE layout (no reference counterpart; built for 16-byte stores and one contiguous
 * page per (block, kv head)): [block][kv_head][K|V][slot][d], and inside each row the
 * 16-byte chunk index is XORed with (slot & 7) so that a page copied verbatim into
 * shared memory can be read without bank conflicts.  Needs d * elem_size % 128 == 0.
 * ============================================================================== */
static inline size_t elem_size(uint32_t dtype) { return dtype == QVO_F32 ? 4 : 2; }

size_t qvo_block_bytes(const qvo_geometry *g) {
    return (size_t)2 * g->block_tokens * g->kv_heads * g->head_dim * elem_size(g->dtype);
}

int qvo_geometry_ok(const qvo_geometry *g) {
    if (!g->block_tokens || !g->kv_heads || !g->head_dim) return 0;
    if (g->dtype > QVO_F16 || g->layout > QVO_LAYOUT_NATIVE) return 0;
    if (g->layout == QVO_LAYOUT_NATIVE && (g->head_dim * elem_size(g->dtype)) % 128 != 0) return 0;
    return 1;
}

/* Byte offset of key (kv=0) or value (kv=1) element (g, i) at pool position
 * `at` = block * B + slot. */
size_t qvo_elem_offset(const qvo_geometry *geo, size_t at, int kv, size_t g, size_t i) {
    size_t B = geo->block_tokens, d = geo->head_dim, kvh = geo->kv_heads;
    size_t e = elem_size(geo->dtype), kv_out = kvh * d;
    size_t b = at / B, slot = at % B;
    if (geo->layout == QVO_LAYOUT_REFERENCE) {
        /* kv_key_word / kv_value_word, discrete.rs:317-329 */
        size_t w = b * (2 * B * kv_out);
        w += kv ? B * kv_out + slot * kv_out + g * d + i : (g * d + i) * B + slot;
        return w * e;
    }
    size_t row = d * e, page = B * row;
    size_t in_row = (i * e) ^ ((slot & 7) << 4);
    return b * (kvh * 2 * page) + g * (2 * page) + (size_t)kv * page + slot * row + in_row;
}

static inline void store_elem(uint8_t *pool, size_t off, uint32_t dtype, float x) {
    if (dtype == QVO_F32) memcpy(pool + off, &x, 4);
    else {
        uint16_t h = dtype == QVO_BF16 ? qvo_f32_to_bf16(x) : qvo_f32_to_f16(x);
        memcpy(pool + off, &h, 2);
    }
}
static inline float load_elem(const uint8_t *pool, size_t off, uint32_t dtype) {
    if (dtype == QVO_F32) { float x; memcpy(&x, pool + off, 4); return x; }
    uint16_t h; memcpy(&h, pool + off, 2);
    return dtype == QVO_BF16 ? qvo_bf16_to_f32(h) : qvo_f16_to_f32(h);
}

/* One position's key (kv=0) or value (kv=1) row of KV head g, widened to f32: the same
 * elements as d calls of load_elem(qvo_elem_offset(..)), with the address arithmetic of a row
 * done once (the reference's kv_key_word / kv_value_word are inlined const fns). */
static void load_row(const uint8_t *pool, const qvo_geometry *geo, size_t at, int kv, size_t g, float *out) {
    size_t B = geo->block_tokens, d = geo->head_dim, kvh = geo->kv_heads, e = elem_size(geo->dtype);
    size_t b = at / B, slot = at % B, kv_out = kvh * d;
    const uint8_t *p;
    size_t stride;
    size_t swz = 0;
    if (geo->layout == QVO_LAYOUT_REFERENCE) {
        size_t w = b * (2 * B * kv_out);
        if (kv) { w += B * kv_out + slot * kv_out + g * d; stride = e; }
        else { w += (g * d) * B + slot; stride = B * e; }
        p = pool + w * e;
    } else {
        size_t row = d * e, page = B * row;
        p = pool + b * (kvh * 2 * page) + g * (2 * page) + (size_t)kv * page + slot * row;
        stride = e;
        swz = (slot & 7) << 4;
    }
    if (geo->dtype == QVO_F32) {
        for (size_t i = 0; i < d; i++) memcpy(out + i, p + ((i * stride) ^ swz), 4);
    } else if (geo->dtype == QVO_BF16) {
        for (size_t i = 0; i < d; i++) { uint16_t h; memcpy(&h, p + ((i * stride) ^ swz), 2); out[i] = qvo_bf16_to_f32(h); }
    } else {
        for (size_t i = 0; i < d; i++) { uint16_t h; memcpy(&h, p + ((i * stride) ^ swz), 2); out[i] = qvo_f16_to_f32(h); }
    }
}

/* The `put` closure, crates/qubivex-backend-cpu/src/sim.rs:377-384: one position's key
 * row and value row (kv_out f32 each) into the pool, narrowed to the pool's dtype. */
static void put(uint8_t *pool, const qvo_geometry *geo, size_t at, const float *k, const float *v) {
    for (size_t g = 0; g < geo->kv_heads; g++)
        for (size_t i = 0; i < geo->head_dim; i++) {
            store_elem(pool, qvo_elem_offset(geo, at, 0, g, i), geo->dtype, k[g * geo->head_dim + i]);
            store_elem(pool, qvo_elem_offset(geo, at, 1, g, i), geo->dtype, v[g * geo->head_dim + i]);
        }
}

/* Validation before any write, crates/qubivex-backend-cpu/src/sim.rs:313-324, :359-376. */
static int validate(const qvo_geometry *geo, size_t pool_blocks, size_t heads, size_t s,
                    const uint32_t *pos, const uint32_t *blocks, size_t n_blocks,
                    const uint32_t *table_at, const uint32_t *sync_to, size_t n_sync) {
    if (!qvo_geometry_ok(geo)) return QVO_ERR_UNSUPPORTED;
    if (heads == 0 || heads % geo->kv_heads != 0) return QVO_ERR_SHAPE;
    size_t B = geo->block_tokens;
    for (size_t i = 0; i < n_blocks; i++)
        if (blocks[i] >= pool_blocks) return QVO_ERR_SHAPE;
    for (size_t i = 0; i < n_sync; i++)
        if (sync_to[i] / B >= pool_blocks) return QVO_ERR_SHAPE;
    for (size_t t = 0; t < s; t++)
        if ((size_t)table_at[t] + pos[t] / B >= n_blocks) return QVO_ERR_SHAPE;
    return QVO_OK;
}

static inline size_t at_of(const qvo_geometry *geo, const uint32_t *blocks,
                           const uint32_t *table_at, size_t t, size_t p) {
    size_t B = geo->block_tokens;
    return (size_t)blocks[table_at[t] + p / B] * B + p % B;
}

/* Sync rows (each 2*kv_out f32: key row then value row) in list order, then every
 * token's new row: crates/qubivex-backend-cpu/src/sim.rs:385-399. */
int qvo_kv_write(uint8_t *pool, size_t pool_blocks, const qvo_geometry *geo, size_t s,
                 const float *k_new, const float *v_new, const uint32_t *pos,
                 const uint32_t *blocks, size_t n_blocks, const uint32_t *table_at,
                 const float *sync, const uint32_t *sync_to, size_t n_sync) {
    int rc = validate(geo, pool_blocks, geo->kv_heads, s, pos, blocks, n_blocks, table_at, sync_to, n_sync);
    if (rc) return rc;
    size_t kv_out = (size_t)geo->kv_heads * geo->head_dim;
    for (size_t r = 0; r < n_sync; r++)
        put(pool, geo, sync_to[r], sync + r * 2 * kv_out, sync + r * 2 * kv_out + kv_out);
    for (size_t t = 0; t < s; t++)
        put(pool, geo, at_of(geo, blocks, table_at, t, pos[t]), k_new + t * kv_out, v_new + t * kv_out);
    return QVO_OK;
}

/* Gather of one token's keys and values per KV head, then `attend` per query head:
 * crates/qubivex-backend-cpu/src/sim.rs:400-429.  q and att are [token][head][d] f32.
 * Tokens [t0, t1) only, so that threads can share the work; one token's result does not
 * depend on any other's. */
static void attend_tokens(const uint8_t *pool, const qvo_geometry *geo, size_t heads,
                          const float *q, const uint32_t *pos, const uint32_t *blocks,
                          const uint32_t *table_at, float *att, size_t t0, size_t t1) {
    size_t d = geo->head_dim, kvh = geo->kv_heads, group = heads / kvh, q_out = heads * d;
    for (size_t t = t0; t < t1; t++) {
        size_t n = (size_t)pos[t] + 1;
        float *ks = malloc(sizeof(float) * n * d * kvh), *vs = malloc(sizeof(float) * n * d * kvh);
        float *scores = malloc(sizeof(float) * n);
        for (size_t p = 0; p < n; p++) {
            size_t to = at_of(geo, blocks, table_at, t, p);
            for (size_t g = 0; g < kvh; g++) {
                load_row(pool, geo, to, 0, g, ks + (g * n + p) * d);
                load_row(pool, geo, to, 1, g, vs + (g * n + p) * d);
            }
        }
        for (size_t hd = 0; hd < heads; hd++) {
            size_t g = hd / group;
            qvo_attend(q + t * q_out + hd * d, ks + g * n * d, vs + g * n * d, d, n - 1,
                       att + t * q_out + hd * d, scores);
        }
        free(ks); free(vs); free(scores);
    }
}

/* The read half of SimDevice::attention (sim.rs:400-429), single thread. */
int qvo_attn_decode(const uint8_t *pool, size_t pool_blocks, const qvo_geometry *geo, size_t heads,
                    size_t s, const float *q, const uint32_t *pos, const uint32_t *blocks,
                    size_t n_blocks, const uint32_t *table_at, float *att) {
    int rc = validate(geo, pool_blocks, heads, s, pos, blocks, n_blocks, table_at, NULL, 0);
    if (rc) return rc;
    attend_tokens(pool, geo, heads, q, pos, blocks, table_at, att, 0, s);
    return QVO_OK;
}

/* The whole op in the reference's order (sim.rs:301-437 without the projections, clip,
 * norms and RoPE, which come before the path): validate, sync rows, new rows, attend. */
int qvo_paged_attention(uint8_t *pool, size_t pool_blocks, const qvo_geometry *geo, size_t heads,
                        size_t s, const float *q, const float *k_new, const float *v_new,
                        const uint32_t *pos, const uint32_t *blocks, size_t n_blocks,
                        const uint32_t *table_at, const float *sync, const uint32_t *sync_to,
                        size_t n_sync, float *att) {
    int rc = validate(geo, pool_blocks, heads, s, pos, blocks, n_blocks, table_at, sync_to, n_sync);
    if (rc) return rc;
    rc = qvo_kv_write(pool, pool_blocks, geo, s, k_new, v_new, pos, blocks, n_blocks, table_at,
                      sync, sync_to, n_sync);
    if (rc) return rc;
    attend_tokens(pool, geo, heads, q, pos, blocks, table_at, att, 0, s);
    return QVO_OK;
}

/* The host path's shape of the same arithmetic: `attend` once per (token, head) on that head's
 * keys and values (crates/qubivex-arch/src/lib.rs:1304-1320, rayon's par_chunks_mut over
 * (token, head)).  The reference's host cache holds each KV head's rows contiguously, so its
 * tasks read them in place; here they live in the paged pool, so a task is one (token, KV head):
 * it gathers that head's rows once and runs `attend` for every query head of the group on them
 * (the gather is not paid once per query head).  Same bits as qvo_attn_decode; `threads` workers
 * take tasks from a shared counter. */
typedef struct {
    const uint8_t *pool; const qvo_geometry *geo; size_t heads, s;
    const float *q; const uint32_t *pos, *blocks, *table_at; float *att;
    size_t next; pthread_mutex_t mu;
} par_job;

static void *par_worker(void *arg) {
    par_job *j = arg;
    size_t d = j->geo->head_dim, kvh = j->geo->kv_heads, group = j->heads / kvh, q_out = j->heads * d;
    float *k = NULL, *v = NULL, *scores = NULL; size_t cap = 0;
    for (;;) {
        pthread_mutex_lock(&j->mu);
        size_t task = j->next++;
        pthread_mutex_unlock(&j->mu);
        if (task >= j->s * kvh) break;
        size_t t = task / kvh, g = task % kvh;
        size_t n = (size_t)j->pos[t] + 1;
        if (n > cap) {
            free(k); free(v); free(scores);
            cap = n; k = malloc(4 * cap * d); v = malloc(4 * cap * d); scores = malloc(4 * cap);
        }
        for (size_t p = 0; p < n; p++) {
            size_t to = at_of(j->geo, j->blocks, j->table_at, t, p);
            load_row(j->pool, j->geo, to, 0, g, k + p * d);
            load_row(j->pool, j->geo, to, 1, g, v + p * d);
        }
        for (size_t hd = g * group; hd < (g + 1) * group; hd++)
            qvo_attend(j->q + t * q_out + hd * d, k, v, d, n - 1, j->att + t * q_out + hd * d, scores);
    }
    free(k); free(v); free(scores);
    return NULL;
}

int qvo_attn_decode_par(const uint8_t *pool, size_t pool_blocks, const qvo_geometry *geo,
                        size_t heads, size_t s, const float *q, const uint32_t *pos,
                        const uint32_t *blocks, size_t n_blocks, const uint32_t *table_at,
                        float *att, int threads) {
    int rc = validate(geo, pool_blocks, heads, s, pos, blocks, n_blocks, table_at, NULL, 0);
    if (rc) return rc;
    par_job j = {pool, geo, heads, s, q, pos, blocks, table_at, att, 0, PTHREAD_MUTEX_INITIALIZER};
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    pthread_t th[256];
    for (int i = 0; i < threads; i++) pthread_create(&th[i], NULL, par_worker, &j);
    for (int i = 0; i < threads; i++) pthread_join(th[i], NULL);
    return QVO_OK;
}

/* Whole-block copies src[i] -> dst[i], in list order: what copy-on-write and compaction
 * do to the pool bytes.  No reference counterpart (the reference copies a whole cache,
 * crates/qubivex-arch/src/lib.rs:409-432, and never moves a block). */
int qvo_block_copy(uint8_t *pool, size_t pool_blocks, const qvo_geometry *geo,
                   const uint32_t *src, const uint32_t *dst, size_t n) {
    if (!qvo_geometry_ok(geo)) return QVO_ERR_UNSUPPORTED;
    size_t bb = qvo_block_bytes(geo);
    for (size_t i = 0; i < n; i++)
        if (src[i] >= pool_blocks || dst[i] >= pool_blocks) return QVO_ERR_SHAPE;
    for (size_t i = 0; i < n; i++)
        if (src[i] != dst[i]) memcpy(pool + dst[i] * bb, pool + src[i] * bb, bb);
    return QVO_OK;
}
