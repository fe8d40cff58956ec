/*
 * CPU oracle for the quantized-weight matmul path of nuclis.
 *
 * TEST INFRASTRUCTURE ONLY. This file restates, in plain C, the arithmetic of
 * the reference engine's CPU path so that the CUDA kernels can be checked
 * against it. Nothing in the shipped library links, loads or calls it; only
 * the tests, the smoke check and the benchmark's CPU-baseline leg do.
 *
 * The reference is Zig and cannot be compiled where this is built, so this is
 * a restatement, pinned bit for bit against the reference's own golden decoder
 * vectors (inference/src/quant/fixtures/{k-affine,k-signed,simple}.json) and
 * its hand-computed unit-test blocks; see tests/test_oracle_golden.py.
 *
 * Build with -O2 -ffp-contract=off: every product and sum below is a separate
 * IEEE operation, as in the reference (no fused multiply-add).
 *
 * What each function follows (paths inside the reference tree):
 *   nu_ref_layout        inference/src/tensor/encoding.zig:29-56
 *   nu_ref_validate_row  inference/src/quant/decode.zig:108-120
 *   nu_ref_row           inference/src/quant/decode.zig:30-103 (ids 0,1,2,6,7,8,10,11,12,13,14,30),
 *                        :147-170 (Q4_K), :198-211 (Q6_K), :432-435 (half)
 *   nu_ref_matvec        inference/src/backends/cpu/root.zig:112-152
 *   nu_ref_gelu/silu     inference/src/backends/cpu/vector.zig:94-98, 178-196
 *   nu_ref_rms_norm      inference/src/backends/cpu/vector.zig:53-64
 *   nu_ref_route         inference/src/backends/cpu/experts.zig:50-79
 *   nu_ref_ffn           inference/src/backends/cpu/experts.zig:107-133
 */
#include <math.h>
#include <pthread.h>
#include <stdatomic.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum {
    NU_REF_OK = 0,
    NU_REF_UNSUPPORTED_ENCODING = 1,
    NU_REF_INVALID_ROW_LENGTH = 2,
    NU_REF_INVALID_BYTE_LENGTH = 3,
    NU_REF_INVALID_SHAPE = 4,
    NU_REF_SCRATCH_TOO_SMALL = 5,
    NU_REF_INVALID_EXPERT = 6,
    NU_REF_NON_FINITE = 7,
};

/* encoding.zig:29-56, restricted to the encodings this path serves. */
int nu_ref_layout(uint32_t id, uint32_t *elements, uint32_t *bytes) {
    uint32_t e, b;
    switch (id) {
    case 0: e = 1; b = 4; break;      /* F32  */
    case 1: e = 1; b = 2; break;      /* F16  */
    case 2: e = 32; b = 18; break;    /* Q4_0 */
    case 6: e = 32; b = 22; break;    /* Q5_0 */
    case 7: e = 32; b = 24; break;    /* Q5_1 */
    case 8: e = 32; b = 34; break;    /* Q8_0 */
    case 10: e = 256; b = 84; break;  /* Q2_K */
    case 11: e = 256; b = 110; break; /* Q3_K */
    case 12: e = 256; b = 144; break; /* Q4_K */
    case 13: e = 256; b = 176; break; /* Q5_K */
    case 14: e = 256; b = 210; break; /* Q6_K */
    case 20: e = 32; b = 18; break;   /* IQ4_NL */
    case 23: e = 256; b = 136; break; /* IQ4_XS */
    case 30: e = 1; b = 2; break;     /* BF16 */
    default: return NU_REF_UNSUPPORTED_ENCODING;
    }
    if (elements) *elements = e;
    if (bytes) *bytes = b;
    return NU_REF_OK;
}

static float half_at(const uint8_t *p);

/* The sixteen values a four-bit IQ4 code selects (decode.zig:437): part of the storage format. */
static const int8_t iq4_values[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

/* decode.zig:73-81: IQ4_NL, 18 bytes per 32 values: d, then 16 bytes whose low nibbles are the first
 * half of the block and whose high nibbles are the second; value = d * table[code]. */
static void iq4nl_block(const uint8_t *block, float *out) {
    const float scale = half_at(block);
    for (int j = 0; j < 16; ++j) {
        out[j] = scale * (float)iq4_values[block[2 + j] & 15u];
        out[j + 16] = scale * (float)iq4_values[block[2 + j] >> 4];
    }
}

/* decode.zig:214-228: IQ4_XS, 136 bytes per 256 values: d, 16 bits of scale high parts, 4 bytes of scale
 * low nibbles, 128 code bytes. Eight groups of 32 with a six-bit scale biased by 32; within a group the
 * low nibbles are the first 16 values and the high nibbles the next 16. */
static void iq4xs_block(const uint8_t *block, float *out) {
    const float d = half_at(block);
    const uint32_t high = (uint32_t)block[2] | ((uint32_t)block[3] << 8);
    for (int g = 0; g < 8; ++g) {
        const uint32_t low = (block[4 + g / 2] >> (4 * (g % 2))) & 15u;
        const int scale = (int)(low | (((high >> (2 * g)) & 3u) << 4)) - 32;
        const float multiplier = d * (float)scale;
        const uint8_t *q = block + 8 + g * 16;
        for (int j = 0; j < 16; ++j) {
            out[g * 32 + j] = multiplier * (float)iq4_values[q[j] & 15u];
            out[g * 32 + j + 16] = multiplier * (float)iq4_values[q[j] >> 4];
        }
    }
}

/* decode.zig:108-120: quotients are compared, nothing is multiplied. */
int nu_ref_validate_row(uint32_t id, size_t byte_count, size_t element_count) {
    uint32_t e, b;
    if (nu_ref_layout(id, &e, &b) != NU_REF_OK) return NU_REF_UNSUPPORTED_ENCODING;
    if (element_count == 0 || element_count % e != 0) return NU_REF_INVALID_ROW_LENGTH;
    if (byte_count % b != 0 || byte_count / b != element_count / e) return NU_REF_INVALID_BYTE_LENGTH;
    return NU_REF_OK;
}

/* decode.zig:432-435: little-endian binary16 widened exactly to binary32. */
static float half_at(const uint8_t *p) {
    uint32_t h = (uint32_t)p[0] | ((uint32_t)p[1] << 8);
    uint32_t sign = (h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 31u;
    uint32_t man = h & 1023u;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalize */
            int shift = 0;
            while (!(man & 1024u)) { man <<= 1; ++shift; }
            man &= 1023u;
            bits = sign | ((uint32_t)(127 - 15 + 1 - shift) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* decode.zig:125-143: Q5_0 (offset = 0: d * (q - 16)) and Q5_1 (d * q + m). Q4_0's nibble order,
 * each code completed by its bit of the 32-bit plane (bit j for value j). */
static void five_block(int offset, const uint8_t *block, float *out) {
    const float d = half_at(block);
    const float m = offset ? half_at(block + 2) : 0.0f;
    const uint8_t *plane = block + (offset ? 4 : 2);
    const uint32_t qh = (uint32_t)plane[0] | ((uint32_t)plane[1] << 8) | ((uint32_t)plane[2] << 16) | ((uint32_t)plane[3] << 24);
    const uint8_t *qs = plane + 4;
    for (int j = 0; j < 16; ++j) {
        const int low = (int)((qs[j] & 15u) | (((qh >> j) & 1u) << 4));
        const int high = (int)((uint32_t)(qs[j] >> 4) | (((qh >> (j + 16)) & 1u) << 4));
        if (offset) {
            out[j] = d * (float)low + m;
            out[j + 16] = d * (float)high + m;
        } else {
            out[j] = d * (float)(low - 16);
            out[j + 16] = d * (float)(high - 16);
        }
    }
}

/* decode.zig:147-170: Q4_K (fifth_bit = 0) and Q5_K (fifth_bit = 1: 32 bytes of high bits at 16, one bit per
 * group in each, the nibbles after them). */
static void q4k_block(int fifth_bit, const uint8_t *block, float *out) {
    const float d = half_at(block);
    const float dmin = half_at(block + 2);
    const uint8_t *sc = block + 4;
    const uint8_t *qs = block + (fifth_bit ? 48 : 16);
    for (int g = 0; g < 8; ++g) {
        uint32_t s, m;
        if (g < 4) {
            s = sc[g] & 63u;
            m = sc[g + 4] & 63u;
        } else {
            s = (sc[g + 4] & 15u) | ((uint32_t)(sc[g - 4] >> 6) << 4);
            m = (uint32_t)(sc[g + 4] >> 4) | ((uint32_t)(sc[g] >> 6) << 4);
        }
        const float multiplier = d * (float)s;
        const float offset = dmin * (float)m;
        for (int c = 0; c < 32; ++c) {
            const uint8_t byte = qs[(g / 2) * 32 + c];
            uint32_t q = (g % 2 == 0) ? (byte & 15u) : (uint32_t)(byte >> 4);
            if (fifth_bit) q |= (((uint32_t)block[16 + c] >> g) & 1u) << 4;
            out[g * 32 + c] = multiplier * (float)q - offset;
        }
    }
}

/* decode.zig:260-275: Q2_K, sixteen groups of 16 two-bit codes, a four-bit scale (low nibble) and a four-bit
 * minimum (high nibble) each under two block scales; each 128-value half packs four bit planes of 32 bytes. */
static void q2k_block(const uint8_t *block, float *out) {
    const float d = half_at(block + 80);
    const float dmin = half_at(block + 82);
    for (int g = 0; g < 16; ++g) {
        const float multiplier = d * (float)(block[g] & 15u);
        const float offset = dmin * (float)(block[g] >> 4);
        for (int c = 0; c < 16; ++c) {
            const int i = g * 16 + c;
            const int shift = 2 * ((i % 128) / 32);
            const uint32_t code = ((uint32_t)block[16 + (i / 128) * 32 + i % 32] >> shift) & 3u;
            out[i] = multiplier * (float)code - offset;
        }
    }
}

/* decode.zig:174-196: Q3_K, biased six-bit scales and an inverted high bit per code (clear means subtract four). */
static void q3k_block(const uint8_t *block, float *out) {
    const float d = half_at(block + 108);
    const uint8_t *scales = block + 96;
    for (int g = 0; g < 16; ++g) {
        const uint32_t nibble = g < 8 ? (scales[g] & 15u) : (uint32_t)(scales[g - 8] >> 4);
        const uint32_t upper = ((uint32_t)scales[8 + g % 4] >> (2 * (g / 4))) & 3u;
        const int scale = (int)(nibble | (upper << 4)) - 32;
        const float multiplier = d * (float)scale;
        for (int c = 0; c < 16; ++c) {
            const int i = g * 16 + c;
            const int low_shift = 2 * ((i % 128) / 32);
            const int low = (int)(((uint32_t)block[32 + (i / 128) * 32 + i % 32] >> low_shift) & 3u);
            const uint32_t nonnegative = ((uint32_t)block[i % 32] >> (i / 32)) & 1u;
            out[i] = multiplier * (float)(low - (nonnegative ? 0 : 4));
        }
    }
}

/* decode.zig:198-211. */
static void q6k_block(const uint8_t *block, float *out) {
    const float d = half_at(block + 208);
    for (int i = 0; i < 256; ++i) {
        const int quarter = (i % 128) / 32;
        const int column = i % 32;
        const int low_shift = (quarter / 2) * 4;
        const int high_shift = quarter * 2;
        const uint32_t low = ((uint32_t)block[(i / 128) * 64 + (quarter % 2) * 32 + column] >> low_shift) & 15u;
        const uint32_t high = ((uint32_t)block[128 + (i / 128) * 32 + column] >> high_shift) & 3u;
        const int value = (int)(low | (high << 4)) - 32;
        const int8_t scale = (int8_t)block[192 + i / 16];
        out[i] = (d * (float)scale) * (float)value;
    }
}

/* decode.zig:30-103, the arms for ids 0, 1, 2, 6, 7, 8, 10, 11, 12, 13, 14, 30. All validation
 * happens before the first write. */
int nu_ref_row(uint32_t id, const uint8_t *bytes, size_t byte_count, float *out, size_t element_count) {
    int rc = nu_ref_validate_row(id, byte_count, element_count);
    if (rc != NU_REF_OK) return rc;
    uint32_t e, b;
    nu_ref_layout(id, &e, &b);
    size_t o = 0;
    for (size_t off = 0; off < byte_count; off += b, o += e) {
        const uint8_t *block = bytes + off;
        switch (id) {
        case 0: {
            uint32_t bits = (uint32_t)block[0] | ((uint32_t)block[1] << 8) | ((uint32_t)block[2] << 16) | ((uint32_t)block[3] << 24);
            memcpy(out + o, &bits, 4);
            break;
        }
        case 1: out[o] = half_at(block); break;
        case 2: {
            /* Q4_0: low nibbles are the first half of the block, high nibbles the second; code - 8 */
            const float scale = half_at(block);
            for (int j = 0; j < 16; ++j) {
                out[o + j] = scale * (float)((int)(block[2 + j] & 15u) - 8);
                out[o + j + 16] = scale * (float)((int)(block[2 + j] >> 4) - 8);
            }
            break;
        }
        case 6: five_block(0, block, out + o); break;
        case 7: five_block(1, block, out + o); break;
        case 8: {
            const float scale = half_at(block);
            for (int j = 0; j < 32; ++j) out[o + j] = scale * (float)(int8_t)block[2 + j];
            break;
        }
        case 10: q2k_block(block, out + o); break;
        case 11: q3k_block(block, out + o); break;
        case 12: q4k_block(0, block, out + o); break;
        case 13: q4k_block(1, block, out + o); break;
        case 14: q6k_block(block, out + o); break;
        case 20: iq4nl_block(block, out + o); break;
        case 23: iq4xs_block(block, out + o); break;
        case 30: {
            uint32_t bits = ((uint32_t)block[0] | ((uint32_t)block[1] << 8)) << 16;
            memcpy(out + o, &bits, 4);
            break;
        }
        }
    }
    return NU_REF_OK;
}

/* ---- matvec: root.zig:112-152 ------------------------------------------- */

typedef struct {
    uint32_t encoding;
    size_t rows, columns, row_bytes;
    const uint8_t *bytes;
    const float *input;
    float *output;
} rows_t;

/* Rows.run, root.zig:144-152: decode the row to F32, widen both operands to
 * F64, sum in column order, round once to F32. */
static int rows_run(const rows_t *r, size_t first, size_t last, float *decoded) {
    for (size_t i = first; i < last; ++i) {
        int rc = nu_ref_row(r->encoding, r->bytes + i * r->row_bytes, r->row_bytes, decoded, r->columns);
        if (rc != NU_REF_OK) return rc;
        double sum = 0;
        for (size_t c = 0; c < r->columns; ++c) sum += (double)decoded[c] * (double)r->input[c];
        r->output[i] = (float)sum;
    }
    return NU_REF_OK;
}

typedef struct {
    const rows_t *rows;
    atomic_size_t *next;
    size_t chunk;
    float *decoded;
    int failure;
} task_t;

/* Rows.task, root.zig:155-164: take chunks from an atomic cursor until none remain. */
static void *task_main(void *arg) {
    task_t *t = (task_t *)arg;
    for (;;) {
        size_t first = atomic_fetch_add_explicit(t->next, t->chunk, memory_order_relaxed);
        if (first >= t->rows->rows) return NULL;
        size_t last = first + t->chunk < t->rows->rows ? first + t->chunk : t->rows->rows;
        int rc = rows_run(t->rows, first, last, t->decoded);
        if (rc != NU_REF_OK) { t->failure = rc; return NULL; }
    }
}

#define NU_REF_MAX_TASKS 64
#define NU_REF_PARALLEL_WEIGHTS ((size_t)1 << 16)
#define NU_REF_CHUNKS_PER_TASK 8

/* matvec, root.zig:112-132. `scratch` holds `scratch_len` floats; as many
 * tasks run as it holds decode rows of `columns`, capped by `max_tasks`
 * (the caller passes the core count it wants used) and 64. The result does
 * not depend on the split. All checks precede any write. */
int nu_ref_matvec(uint32_t encoding, size_t rows, size_t columns, const uint8_t *bytes, size_t byte_count,
                  const float *input, size_t input_len, float *output, size_t output_len,
                  float *scratch, size_t scratch_len, unsigned max_tasks) {
    if (rows == 0 || columns == 0 || input_len != columns || output_len != rows) return NU_REF_INVALID_SHAPE;
    if (scratch_len < columns) return NU_REF_SCRATCH_TOO_SMALL;
    if (byte_count % rows != 0) return NU_REF_INVALID_BYTE_LENGTH;
    const size_t row_bytes = byte_count / rows;
    int rc = nu_ref_validate_row(encoding, row_bytes, columns);
    if (rc != NU_REF_OK) return rc;
    size_t weights;
    if (__builtin_mul_overflow(rows, columns, &weights)) weights = SIZE_MAX;
    size_t tasks = 1;
    if (weights >= NU_REF_PARALLEL_WEIGHTS) {
        tasks = max_tasks ? max_tasks : 1;
        if (tasks > NU_REF_MAX_TASKS) tasks = NU_REF_MAX_TASKS;
        if (tasks > rows) tasks = rows;
        if (tasks > scratch_len / columns) tasks = scratch_len / columns;
    }
    rows_t r = { encoding, rows, columns, row_bytes, bytes, input, output };
    if (tasks <= 1) return rows_run(&r, 0, rows, scratch);
    atomic_size_t next = 0;
    size_t chunk = rows / (tasks * NU_REF_CHUNKS_PER_TASK);
    if (chunk < 1) chunk = 1;
    pthread_t threads[NU_REF_MAX_TASKS];
    task_t ctx[NU_REF_MAX_TASKS];
    size_t started = 0;
    for (size_t t = 0; t < tasks; ++t) ctx[t] = (task_t){ &r, &next, chunk, scratch + t * columns, NU_REF_OK };
    for (size_t t = 0; t + 1 < tasks; ++t) { /* the caller's thread is the last task */
        if (pthread_create(&threads[t], NULL, task_main, &ctx[t]) != 0) break;
        ++started;
    }
    task_main(&ctx[tasks - 1]);
    /* If a thread failed to start its share is still taken: the cursor is shared. */
    for (size_t t = 0; t < started; ++t) pthread_join(threads[t], NULL);
    for (size_t t = 0; t < tasks; ++t) if (ctx[t].failure != NU_REF_OK) return ctx[t].failure;
    return NU_REF_OK;
}

/* ---- activations: vector.zig:94-98, 178-196 ------------------------------ */

float nu_ref_gelu(float x) {
    const double v = x;
    const double inner = 0.7978845608028654 * v * (1.0 + 0.044715 * v * v);
    return (float)(0.5 * v * (1.0 + tanh(inner)));
}

static double logistic(float x) {
    const double wide = x;
    if (wide >= 0) return 1 / (1 + exp(-wide));
    const double e = exp(wide);
    return e / (1 + e);
}

float nu_ref_silu(float x) {
    if (isinf(x) && x < 0) return -0.0f;
    return (float)((double)x * logistic(x));
}

/* ---- rmsNorm: backends/cpu/vector.zig:53-64 (F64 sum of squares, one division per element) ---- */

int nu_ref_rms_norm(const float *input, float *output, size_t n, float epsilon) {
    if (n == 0 || !isfinite(epsilon) || epsilon <= 0) return NU_REF_INVALID_SHAPE;
    double squares = 0;
    for (size_t i = 0; i < n; ++i) {
        if (!isfinite(input[i])) return NU_REF_INVALID_SHAPE;
        squares += (double)input[i] * (double)input[i];
    }
    const double denominator = sqrt(squares / (double)n + (double)epsilon);
    for (size_t i = 0; i < n; ++i) output[i] = (float)((double)input[i] / denominator);
    return NU_REF_OK;
}

/* ---- routing: experts.zig:50-79 ------------------------------------------ */

#define NU_REF_MAX_EXPERTS 1024
#define NU_REF_WEIGHT_SUM_FLOOR 6.103515625e-5

int nu_ref_route(const float *logits, size_t experts, uint32_t *indices, float *weights, size_t k) {
    if (k == 0 || k > experts) return NU_REF_INVALID_SHAPE;
    double maximum = -INFINITY;
    for (size_t i = 0; i < experts; ++i) {
        if (!isfinite(logits[i])) return NU_REF_NON_FINITE;
        if ((double)logits[i] > maximum) maximum = logits[i];
    }
    double total = 0;
    for (size_t i = 0; i < experts; ++i) total += exp((double)logits[i] - maximum);
    if (experts > NU_REF_MAX_EXPERTS) return NU_REF_INVALID_SHAPE;
    unsigned char taken[NU_REF_MAX_EXPERTS];
    memset(taken, 0, sizeof taken);
    double selected_sum = 0;
    for (size_t slot = 0; slot < k; ++slot) {
        size_t best = experts;
        for (size_t i = 0; i < experts; ++i) {
            if (taken[i]) continue;
            if (best == experts || logits[i] > logits[best]) best = i;
        }
        taken[best] = 1;
        indices[slot] = (uint32_t)best;
        const double probability = exp((double)logits[best] - maximum) / total;
        weights[slot] = (float)probability;
        selected_sum += probability;
    }
    const double denominator = selected_sum > NU_REF_WEIGHT_SUM_FLOOR ? selected_sum : NU_REF_WEIGHT_SUM_FLOOR;
    for (size_t s = 0; s < k; ++s) weights[s] = (float)((double)weights[s] / denominator);
    return NU_REF_OK;
}

/* ---- gathered expert FFN: experts.zig:20-43, 107-133 ---------------------- */

static int expert_bytes(uint32_t encoding, size_t experts, size_t rows, size_t columns, size_t byte_count, size_t *per_expert) {
    if (experts == 0 || rows == 0 || columns == 0) return NU_REF_INVALID_SHAPE;
    if (byte_count % experts != 0) return NU_REF_INVALID_BYTE_LENGTH;
    const size_t per = byte_count / experts;
    if (per % rows != 0) return NU_REF_INVALID_BYTE_LENGTH;
    int rc = nu_ref_validate_row(encoding, per / rows, columns);
    if (rc != NU_REF_OK) return rc;
    *per_expert = per;
    return NU_REF_OK;
}

/* output = sum_s weights[s] * scale[e_s] * down[e_s] * (gelu(g) (.) u), (g, u)
 * the halves of gate_up[e_s] * input; slots in order, F64 accumulator.
 * `down_scale` may be NULL. Scratch and accumulator are allocated here (the
 * reference borrows them from its caller); that changes no arithmetic. */
int nu_ref_ffn(uint32_t gu_encoding, size_t gu_experts, size_t gu_rows, size_t gu_columns, const uint8_t *gu_bytes, size_t gu_byte_count,
               uint32_t dn_encoding, size_t dn_experts, size_t dn_rows, size_t dn_columns, const uint8_t *dn_bytes, size_t dn_byte_count,
               const float *down_scale, size_t down_scale_len,
               const float *input, size_t input_len, const uint32_t *indices, const float *weights, size_t slots,
               float *output, size_t output_len, unsigned max_tasks) {
    size_t gu_per, dn_per;
    int rc = expert_bytes(gu_encoding, gu_experts, gu_rows, gu_columns, gu_byte_count, &gu_per);
    if (rc != NU_REF_OK) return rc;
    rc = expert_bytes(dn_encoding, dn_experts, dn_rows, dn_columns, dn_byte_count, &dn_per);
    if (rc != NU_REF_OK) return rc;
    if (gu_experts != dn_experts || gu_rows != 2 * dn_columns || gu_columns != input_len || dn_rows != output_len) return NU_REF_INVALID_SHAPE;
    if (slots == 0) return NU_REF_INVALID_SHAPE;
    if (down_scale && down_scale_len != dn_experts) return NU_REF_INVALID_SHAPE;
    for (size_t s = 0; s < slots; ++s) if (indices[s] >= gu_experts) return NU_REF_INVALID_EXPERT;
    for (size_t s = 0; s < slots; ++s) if (!isfinite(weights[s])) return NU_REF_NON_FINITE;
    const size_t ff = dn_columns;
    const size_t widest = gu_columns > dn_columns ? gu_columns : dn_columns;
    const size_t tasks = max_tasks ? (max_tasks > NU_REF_MAX_TASKS ? NU_REF_MAX_TASKS : max_tasks) : 1;
    float *gate_up_row = (float *)malloc(sizeof(float) * (gu_rows + ff + dn_rows + widest * tasks));
    double *acc = (double *)calloc(output_len, sizeof(double));
    if (!gate_up_row || !acc) { free(gate_up_row); free(acc); return NU_REF_SCRATCH_TOO_SMALL; }
    float *hidden = gate_up_row + gu_rows;
    float *projected = hidden + ff;
    float *decode = projected + dn_rows;
    for (size_t s = 0; s < slots && rc == NU_REF_OK; ++s) {
        const uint32_t e = indices[s];
        rc = nu_ref_matvec(gu_encoding, gu_rows, gu_columns, gu_bytes + (size_t)e * gu_per, gu_per, input, input_len, gate_up_row, gu_rows, decode, widest * tasks, (unsigned)tasks);
        if (rc != NU_REF_OK) break;
        for (size_t i = 0; i < ff; ++i) hidden[i] = nu_ref_gelu(gate_up_row[i]) * gate_up_row[ff + i];
        rc = nu_ref_matvec(dn_encoding, dn_rows, dn_columns, dn_bytes + (size_t)e * dn_per, dn_per, hidden, ff, projected, dn_rows, decode, widest * tasks, (unsigned)tasks);
        if (rc != NU_REF_OK) break;
        const double scale = down_scale ? (double)down_scale[e] : 1.0;
        for (size_t i = 0; i < output_len; ++i) acc[i] += (double)weights[s] * (scale * (double)projected[i]);
    }
    if (rc == NU_REF_OK) for (size_t i = 0; i < output_len; ++i) output[i] = (float)acc[i];
    free(gate_up_row);
    free(acc);
    return rc;
}

/* Per-element magnitude sum_c |w[r,c] * x[c]| in F64: the scale of the
 * reference's acceptance formula 4e-6 * sum|w*x| + 1e-6
 * (inference/metal-check.zig:3976). Not part of the engine; test support. */
int nu_ref_matvec_abs(uint32_t encoding, size_t rows, size_t columns, const uint8_t *bytes, size_t byte_count,
                      const float *input, double *output) {
    if (rows == 0 || columns == 0 || byte_count % rows != 0) return NU_REF_INVALID_SHAPE;
    const size_t row_bytes = byte_count / rows;
    int rc = nu_ref_validate_row(encoding, row_bytes, columns);
    if (rc != NU_REF_OK) return rc;
    float *decoded = (float *)malloc(sizeof(float) * columns);
    if (!decoded) return NU_REF_SCRATCH_TOO_SMALL;
    for (size_t r = 0; r < rows; ++r) {
        nu_ref_row(encoding, bytes + r * row_bytes, row_bytes, decoded, columns);
        double sum = 0;
        for (size_t c = 0; c < columns; ++c) sum += fabs((double)decoded[c] * (double)input[c]);
        output[r] = sum;
    }
    free(decoded);
    return NU_REF_OK;
}
