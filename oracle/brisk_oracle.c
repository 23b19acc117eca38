/* TEST INFRASTRUCTURE, NOT PRODUCT CODE - see brisk_oracle.h.
 *
 * A plain-C restatement of what the reference CPU engine computes on the token loop, written
 * from its algorithm, operation by operation, so that float rounding happens at the same places:
 * compiled with -ffp-contract=off and without fast-math, like the reference's Release build on
 * x86-64 (no FMA contraction there). Each function cites the reference code it restates, by the
 * file's path inside the brisk-llm project.
 *
 * The model description structs point at caller-owned host memory that must outlive the session.
 */
#include "brisk_oracle.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define QK 32   /* values per Q4_0 / Q8_0 block      (src/quant.h:12)  */
#define QKK 256 /* values per K-quant / TQ2_0 block  (src/quant.h:89)  */

static _Thread_local char g_error[256];
static void set_error(const char* what) { snprintf(g_error, sizeof(g_error), "%s", what); }
const char* oracle_last_error(void) { return g_error; }

/* ---- a minimal fork-join helper (each index is computed by exactly one thread, so results do not
 * depend on the thread count - the property the reference's thread pool also has) ---- */
#include <pthread.h>
#include <unistd.h>

typedef void (*range_fn)(void* ctx, int64_t begin, int64_t end);
typedef struct { range_fn fn; void* ctx; int64_t begin, end; } range_job;
static void* range_thread(void* p) {
    range_job* j = (range_job*)p;
    j->fn(j->ctx, j->begin, j->end);
    return NULL;
}
static int oracle_threads(void) {
    const char* env = getenv("BRISK_ORACLE_THREADS");
    long n = env ? atol(env) : sysconf(_SC_NPROCESSORS_ONLN);
    return n < 1 ? 1 : (n > 256 ? 256 : (int)n);
}
static void parallel_for(int64_t n, range_fn fn, void* ctx) {
    int threads = oracle_threads();
    if (threads > n) threads = (int)n;
    if (threads <= 1) {
        fn(ctx, 0, n);
        return;
    }
    pthread_t tid[256];
    range_job jobs[256];
    for (int i = 0; i < threads; ++i) {
        jobs[i].fn = fn;
        jobs[i].ctx = ctx;
        jobs[i].begin = n * i / threads;
        jobs[i].end = n * (i + 1) / threads;
        if (i > 0) pthread_create(&tid[i], NULL, range_thread, &jobs[i]);
    }
    range_thread(&jobs[0]);
    for (int i = 1; i < threads; ++i) pthread_join(tid[i], NULL);
}

/* ---- half <-> float (src/quant.cpp:61-113): bit manipulation, round to nearest even ---- */

float oracle_half_to_float(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16, e = (h >> 10) & 0x1Fu, m = h & 0x3FFu, bits;
    if (e == 0x1F) {
        bits = sign | 0x7F800000u | (m << 13);
    } else if (e != 0) {
        bits = sign | ((e + 112u) << 23) | (m << 13);
    } else if (m != 0) {
        e = 113;
        while (!(m & 0x400u)) {
            m <<= 1;
            --e;
        }
        bits = sign | (e << 23) | ((m & 0x3FFu) << 13);
    } else {
        bits = sign;
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t oracle_float_to_half(float f) {
    uint32_t bits;
    memcpy(&bits, &f, 4);
    uint32_t sign = (bits >> 16) & 0x8000u, m = bits & 0x7FFFFFu, be = (bits >> 23) & 0xFFu;
    int32_t e = (int32_t)be - 127 + 15;
    if (be == 0xFF) return (uint16_t)(sign | 0x7C00u | (m ? 0x200u : 0u));
    if (e >= 0x1F) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        m |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - e), half = m >> shift, rem = m & ((1u << shift) - 1u), mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1u))) ++half;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((uint32_t)e << 10) | (m >> 13), rem = m & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) ++half;
    return (uint16_t)(sign | half);
}

/* ---- block layouts (src/quant.h:26-130, :199-204), packed exactly as in a GGUF file ---- */
#pragma pack(push, 1)
typedef struct { uint16_t d; uint8_t qs[16]; } q4_0_t;                               /* 18 B  */
typedef struct { uint16_t d, m; uint8_t qs[16]; } q4_1_t;                            /* 20 B  */
typedef struct { uint16_t d; uint8_t qh[4]; uint8_t qs[16]; } q5_0_t;                /* 22 B  */
typedef struct { uint16_t d; int8_t qs[32]; } q8_0_t;                                /* 34 B  */
typedef struct { uint16_t d, dmin; uint8_t scales[12]; uint8_t qh[32]; uint8_t qs[128]; } q5_k_t; /* 176 B */
typedef struct { uint16_t d, dmin; uint8_t scales[12]; uint8_t qs[128]; } q4_k_t;    /* 144 B */
typedef struct { uint8_t ql[128]; uint8_t qh[64]; int8_t scales[16]; uint16_t d; } q6_k_t; /* 210 B */
typedef struct { uint8_t qs[64]; uint16_t d; } tq2_0_t;                              /* 66 B  */
typedef struct { float d; int8_t qs[256]; int16_t bsums[16]; } q8_k_t;               /* 292 B */
#pragma pack(pop)

static size_t type_block_elems(int32_t t) {
    switch (t) {
        case BRISK_TYPE_Q4_0: case BRISK_TYPE_Q4_1: case BRISK_TYPE_Q5_0: case BRISK_TYPE_Q8_0: return QK;
        case BRISK_TYPE_Q4_K: case BRISK_TYPE_Q5_K: case BRISK_TYPE_Q6_K: case BRISK_TYPE_TQ2_0: return QKK;
        default: return 1;
    }
}
static size_t type_block_bytes(int32_t t) {
    switch (t) {
        case BRISK_TYPE_F32: return 4;
        case BRISK_TYPE_F16: case BRISK_TYPE_BF16: return 2;
        case BRISK_TYPE_Q4_0: return 18;
        case BRISK_TYPE_Q4_1: return 20;
        case BRISK_TYPE_Q5_0: return 22;
        case BRISK_TYPE_Q5_K: return 176;
        case BRISK_TYPE_Q8_0: return 34;
        case BRISK_TYPE_Q4_K: return 144;
        case BRISK_TYPE_Q6_K: return 210;
        case BRISK_TYPE_TQ2_0: return 66;
        default: return 0;
    }
}
static int type_takes_q8_k(int32_t t) { return t == BRISK_TYPE_Q4_K || t == BRISK_TYPE_Q5_K || t == BRISK_TYPE_Q6_K || t == BRISK_TYPE_TQ2_0; }
static int type_is_float(int32_t t) { return t == BRISK_TYPE_F32 || t == BRISK_TYPE_F16 || t == BRISK_TYPE_BF16; }
/* src/model.cpp:20-25 */
static float bfloat_to_float(uint16_t b) {
    const uint32_t bits = (uint32_t)b << 16;
    float out;
    memcpy(&out, &bits, sizeof out);
    return out;
}

/* ---- activation quantisers ---- */

/* src/quant.cpp:115-142 (scalar branch): d = amax/127 kept unrounded for the division, stored as half. */
void oracle_quantize_q8_0(const float* x, void* out, uint64_t count) {
    q8_0_t* y = (q8_0_t*)out;
    for (uint64_t b = 0; b < count / QK; ++b) {
        const float* v = x + b * QK;
        float amax = 0.0f;
        for (int i = 0; i < QK; ++i) amax = fmaxf(amax, fabsf(v[i]));
        const float d = amax / 127.0f;
        const float inv = d != 0.0f ? 1.0f / d : 0.0f;
        y[b].d = oracle_float_to_half(d);
        for (int i = 0; i < QK; ++i) y[b].qs[i] = (int8_t)nearbyintf(v[i] * inv);
    }
}

/* src/quant.cpp:146-194 (scalar branch, 8 bits): scale by the signed extreme so it maps to -127;
 * d = 1/inverse in f32; values capped at 127; sums of each 16 values. */
void oracle_quantize_q8_k(const float* x, void* out, uint64_t count) {
    q8_k_t* y = (q8_k_t*)out;
    for (uint64_t b = 0; b < count / QKK; ++b) {
        const float* v = x + b * QKK;
        float max = 0.0f, amax = 0.0f;
        for (int i = 0; i < QKK; ++i) {
            const float ax = fabsf(v[i]);
            if (ax > amax) {
                amax = ax;
                max = v[i];
            }
        }
        if (amax == 0.0f) {
            memset(&y[b], 0, sizeof(q8_k_t));
            continue;
        }
        const float inv = -127.0f / max;
        y[b].d = 1.0f / inv;
        for (int i = 0; i < QKK; ++i) y[b].qs[i] = (int8_t)fminf(127.0f, nearbyintf(inv * v[i]));
        for (int g = 0; g < 16; ++g) {
            int sum = 0;
            for (int i = 0; i < 16; ++i) sum += y[b].qs[g * 16 + i];
            y[b].bsums[g] = (int16_t)sum;
        }
    }
}

/* ---- weight decoders ---- */

/* 6-bit scale and minimum of sub-block j of a Q4_K block (src/quant.h:256-264). */
static void q4_k_scale_min(const uint8_t* s, int j, uint8_t* sc, uint8_t* mn) {
    if (j < 4) {
        *sc = s[j] & 63;
        *mn = s[j + 4] & 63;
    } else {
        *sc = (uint8_t)((s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4));
        *mn = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

/* The 256 six-bit values of a Q6_K block minus 32, in weight order (src/quant.cpp:285-297). */
static void q6_k_unpack(const q6_k_t* b, int8_t* q) {
    for (int half = 0; half < 2; ++half) {
        const uint8_t* ql = b->ql + half * 64;
        const uint8_t* qh = b->qh + half * 32;
        int8_t* y = q + half * 128;
        for (int l = 0; l < 32; ++l) {
            y[l] = (int8_t)(((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32);
            y[l + 32] = (int8_t)(((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32);
            y[l + 64] = (int8_t)(((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32);
            y[l + 96] = (int8_t)(((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32);
        }
    }
}

/* dequantize_q4_0 :196, _q4_1 :207, _q5_0 :219, _q8_0 :234, _q4_k :241, _q5_k :263, _q6_k :299, _tq2_0 :565 (src/quant.cpp). */
int oracle_dequantize(int32_t type, const void* blocks, float* out, uint64_t count) {
    switch (type) {
        case BRISK_TYPE_F32: memcpy(out, blocks, count * 4); return 0;
        case BRISK_TYPE_F16:
            for (uint64_t i = 0; i < count; ++i) out[i] = oracle_half_to_float(((const uint16_t*)blocks)[i]);
            return 0;
        case BRISK_TYPE_Q4_0: {
            const q4_0_t* w = (const q4_0_t*)blocks;
            for (uint64_t b = 0; b < count / QK; ++b) {
                const float d = oracle_half_to_float(w[b].d);
                for (int i = 0; i < 16; ++i) {
                    out[b * QK + i] = (float)((w[b].qs[i] & 0xF) - 8) * d;
                    out[b * QK + i + 16] = (float)((w[b].qs[i] >> 4) - 8) * d;
                }
            }
            return 0;
        }
        case BRISK_TYPE_BF16:
            for (uint64_t i = 0; i < count; ++i) out[i] = bfloat_to_float(((const uint16_t*)blocks)[i]);
            return 0;
        case BRISK_TYPE_Q4_1: {
            const q4_1_t* w = (const q4_1_t*)blocks;
            for (uint64_t b = 0; b < count / QK; ++b) {
                const float d = oracle_half_to_float(w[b].d), m = oracle_half_to_float(w[b].m);
                for (int i = 0; i < 16; ++i) {
                    out[b * QK + i] = (float)(w[b].qs[i] & 0xF) * d + m;
                    out[b * QK + i + 16] = (float)(w[b].qs[i] >> 4) * d + m;
                }
            }
            return 0;
        }
        case BRISK_TYPE_Q5_0: {
            const q5_0_t* w = (const q5_0_t*)blocks;
            for (uint64_t b = 0; b < count / QK; ++b) {
                const float d = oracle_half_to_float(w[b].d);
                uint32_t qh;
                memcpy(&qh, w[b].qh, 4);
                for (int i = 0; i < 16; ++i) {
                    const int lo = (w[b].qs[i] & 0xF) | (int)(((qh >> i) & 1) << 4);
                    const int hi = (w[b].qs[i] >> 4) | (int)(((qh >> (i + 16)) & 1) << 4);
                    out[b * QK + i] = (float)(lo - 16) * d;
                    out[b * QK + i + 16] = (float)(hi - 16) * d;
                }
            }
            return 0;
        }
        case BRISK_TYPE_Q8_0: {
            const q8_0_t* w = (const q8_0_t*)blocks;
            for (uint64_t b = 0; b < count / QK; ++b) {
                const float d = oracle_half_to_float(w[b].d);
                for (int i = 0; i < QK; ++i) out[b * QK + i] = (float)w[b].qs[i] * d;
            }
            return 0;
        }
        case BRISK_TYPE_Q5_K: {
            const q5_k_t* w = (const q5_k_t*)blocks;
            for (uint64_t b = 0; b < count / QKK; ++b) {
                const float d = oracle_half_to_float(w[b].d), dmin = oracle_half_to_float(w[b].dmin);
                float* y = out + b * QKK;
                for (int chunk = 0; chunk < 4; ++chunk) {
                    uint8_t sc, mn;
                    q4_k_scale_min(w[b].scales, 2 * chunk, &sc, &mn);
                    const float d1 = d * sc, m1 = dmin * mn;
                    q4_k_scale_min(w[b].scales, 2 * chunk + 1, &sc, &mn);
                    const float d2 = d * sc, m2 = dmin * mn;
                    const uint8_t* q = w[b].qs + chunk * 32;
                    const uint8_t lo_bit = (uint8_t)(1u << (2 * chunk)), hi_bit = (uint8_t)(lo_bit << 1);
                    for (int i = 0; i < 32; ++i) {
                        y[chunk * 64 + i] = d1 * (float)((q[i] & 0xF) | ((w[b].qh[i] & lo_bit) ? 16 : 0)) - m1;
                        y[chunk * 64 + 32 + i] = d2 * (float)((q[i] >> 4) | ((w[b].qh[i] & hi_bit) ? 16 : 0)) - m2;
                    }
                }
            }
            return 0;
        }
        case BRISK_TYPE_Q4_K: {
            const q4_k_t* w = (const q4_k_t*)blocks;
            for (uint64_t b = 0; b < count / QKK; ++b) {
                const float d = oracle_half_to_float(w[b].d), dmin = oracle_half_to_float(w[b].dmin);
                float* y = out + b * QKK;
                for (int chunk = 0; chunk < 4; ++chunk) {
                    uint8_t sc, mn;
                    q4_k_scale_min(w[b].scales, 2 * chunk, &sc, &mn);
                    const float d1 = d * sc, m1 = dmin * mn;
                    q4_k_scale_min(w[b].scales, 2 * chunk + 1, &sc, &mn);
                    const float d2 = d * sc, m2 = dmin * mn;
                    const uint8_t* q = w[b].qs + chunk * 32;
                    for (int i = 0; i < 32; ++i) {
                        y[chunk * 64 + i] = d1 * (float)(q[i] & 0xF) - m1;
                        y[chunk * 64 + 32 + i] = d2 * (float)(q[i] >> 4) - m2;
                    }
                }
            }
            return 0;
        }
        case BRISK_TYPE_Q6_K: {
            const q6_k_t* w = (const q6_k_t*)blocks;
            int8_t q[QKK];
            for (uint64_t b = 0; b < count / QKK; ++b) {
                const float d = oracle_half_to_float(w[b].d);
                q6_k_unpack(&w[b], q);
                for (int i = 0; i < QKK; ++i) out[b * QKK + i] = d * w[b].scales[i / 16] * q[i];
            }
            return 0;
        }
        case BRISK_TYPE_TQ2_0: {
            const tq2_0_t* w = (const tq2_0_t*)blocks;
            for (uint64_t b = 0; b < count / QKK; ++b) {
                const float d = oracle_half_to_float(w[b].d);
                float* y = out + b * QKK;
                for (int j = 0; j < 64; j += 32)
                    for (int l = 0; l < 4; ++l)
                        for (int m = 0; m < 32; ++m) *y++ = (float)(((w[b].qs[j + m] >> (2 * l)) & 3) - 1) * d;
            }
            return 0;
        }
        default: return -1;
    }
}

/* ---- row dot products: integer block dots, f32 scaling, f32 running sum over blocks in order ---- */

/* src/quant.cpp:445-456 */
static float dot_q4_0(const q4_0_t* w, const q8_0_t* x, size_t blocks) {
    float sum = 0.0f;
    for (size_t b = 0; b < blocks; ++b) {
        int32_t acc = 0;
        for (int i = 0; i < 16; ++i) {
            acc += ((w[b].qs[i] & 0xF) - 8) * x[b].qs[i];
            acc += ((w[b].qs[i] >> 4) - 8) * x[b].qs[i + 16];
        }
        sum += (float)acc * oracle_half_to_float(w[b].d) * oracle_half_to_float(x[b].d);
    }
    return sum;
}

/* src/quant.cpp:458-472 */
static float dot_q5_0(const q5_0_t* w, const q8_0_t* x, size_t blocks) {
    float sum = 0.0f;
    for (size_t b = 0; b < blocks; ++b) {
        uint32_t qh;
        memcpy(&qh, w[b].qh, 4);
        int32_t acc = 0;
        for (int i = 0; i < 16; ++i) {
            const int lo = ((w[b].qs[i] & 0xF) | (int)(((qh >> i) & 1) << 4)) - 16;
            const int hi = ((w[b].qs[i] >> 4) | (int)(((qh >> (i + 16)) & 1) << 4)) - 16;
            acc += lo * x[b].qs[i] + hi * x[b].qs[i + 16];
        }
        sum += (float)acc * oracle_half_to_float(w[b].d) * oracle_half_to_float(x[b].d);
    }
    return sum;
}

/* src/quant.cpp:484-498: the offset m multiplies the activation block's sum, scaled by the activation scale first. */
static float dot_q4_1(const q4_1_t* w, const q8_0_t* x, size_t blocks) {
    float sum = 0.0f;
    for (size_t b = 0; b < blocks; ++b) {
        int32_t acc = 0, xsum = 0;
        for (int i = 0; i < 16; ++i) {
            acc += (w[b].qs[i] & 0xF) * x[b].qs[i];
            acc += (w[b].qs[i] >> 4) * x[b].qs[i + 16];
            xsum += x[b].qs[i] + x[b].qs[i + 16];
        }
        const float dx = oracle_half_to_float(x[b].d);
        sum += (float)acc * oracle_half_to_float(w[b].d) * dx + oracle_half_to_float(w[b].m) * (dx * (float)xsum);
    }
    return sum;
}

/* src/quant.cpp:523-547: Q4_K's arithmetic with the fifth bit of every weight taken from qh. */
static float dot_q5_k(const q5_k_t* w, const q8_k_t* x, size_t blocks) {
    float sum = 0.0f;
    for (size_t b = 0; b < blocks; ++b) {
        int32_t weighted = 0, offsets = 0;
        for (int sb = 0; sb < 8; ++sb) {
            uint8_t sc, mn;
            q4_k_scale_min(w[b].scales, sb, &sc, &mn);
            const uint8_t* q = w[b].qs + (sb / 2) * 32;
            const uint8_t bit = (uint8_t)(1u << sb);
            const int8_t* xq = x[b].qs + sb * 32;
            int32_t dot = 0;
            for (int i = 0; i < 32; ++i) {
                const int v = ((sb & 1) ? (q[i] >> 4) : (q[i] & 0xF)) | ((w[b].qh[i] & bit) ? 16 : 0);
                dot += v * xq[i];
            }
            weighted += sc * dot;
            offsets += mn * (x[b].bsums[2 * sb] + x[b].bsums[2 * sb + 1]);
        }
        sum += x[b].d * (oracle_half_to_float(w[b].d) * (float)weighted - oracle_half_to_float(w[b].dmin) * (float)offsets);
    }
    return sum;
}

/* src/quant.cpp:474-482 */
static float dot_q8_0(const q8_0_t* w, const q8_0_t* x, size_t blocks) {
    float sum = 0.0f;
    for (size_t b = 0; b < blocks; ++b) {
        int32_t acc = 0;
        for (int i = 0; i < QK; ++i) acc += w[b].qs[i] * x[b].qs[i];
        sum += (float)acc * oracle_half_to_float(w[b].d) * oracle_half_to_float(x[b].d);
    }
    return sum;
}

/* src/quant.cpp:500-521: sum_sb scale*dot and sum_sb min*sum(x) as integers, one f32 expression per block. */
static float dot_q4_k(const q4_k_t* w, const q8_k_t* x, size_t blocks) {
    float sum = 0.0f;
    for (size_t b = 0; b < blocks; ++b) {
        int32_t weighted = 0, offsets = 0;
        for (int sb = 0; sb < 8; ++sb) {
            uint8_t sc, mn;
            q4_k_scale_min(w[b].scales, sb, &sc, &mn);
            const uint8_t* q = w[b].qs + (sb / 2) * 32;
            const int8_t* xq = x[b].qs + sb * 32;
            int32_t dot = 0;
            for (int i = 0; i < 32; ++i) dot += ((sb & 1) ? (q[i] >> 4) : (q[i] & 0xF)) * xq[i];
            weighted += sc * dot;
            offsets += mn * (x[b].bsums[2 * sb] + x[b].bsums[2 * sb + 1]);
        }
        sum += x[b].d * (oracle_half_to_float(w[b].d) * (float)weighted - oracle_half_to_float(w[b].dmin) * (float)offsets);
    }
    return sum;
}

/* src/quant.cpp:549-563 */
static float dot_q6_k(const q6_k_t* w, const q8_k_t* x, size_t blocks) {
    int8_t q[QKK];
    float sum = 0.0f;
    for (size_t b = 0; b < blocks; ++b) {
        q6_k_unpack(&w[b], q);
        int32_t weighted = 0;
        for (int g = 0; g < 16; ++g) {
            int32_t dot = 0;
            for (int i = 0; i < 16; ++i) dot += q[g * 16 + i] * x[b].qs[g * 16 + i];
            weighted += w[b].scales[g] * dot;
        }
        sum += x[b].d * oracle_half_to_float(w[b].d) * (float)weighted;
    }
    return sum;
}

/* src/quant.cpp:580-596: sum((q-1) x) = sum(q x) - sum(x) with sum(x) from the block sums. */
static float dot_tq2_0(const tq2_0_t* w, const q8_k_t* x, size_t blocks) {
    float sum = 0.0f;
    for (size_t b = 0; b < blocks; ++b) {
        int32_t acc = 0;
        int i = 0;
        for (int j = 0; j < 64; j += 32)
            for (int l = 0; l < 4; ++l)
                for (int m = 0; m < 32; ++m) acc += ((w[b].qs[j + m] >> (2 * l)) & 3) * x[b].qs[i++];
        int32_t xsum = 0;
        for (int g = 0; g < 16; ++g) xsum += x[b].bsums[g];
        sum += x[b].d * oracle_half_to_float(w[b].d) * (float)(acc - xsum);
    }
    return sum;
}

/* src/kernels_f32.cpp:231-242 (non-NEON branch): 16 partial sums, tail, then the lanes in order. */
static float dot_f32(const float* a, const float* b, size_t n) {
    float lanes[16] = {0};
    size_t i = 0;
    for (; i + 16 <= n; i += 16)
        for (int j = 0; j < 16; ++j) lanes[j] += a[i + j] * b[i + j];
    float sum = 0.0f;
    for (; i < n; ++i) sum += a[i] * b[i];
    for (int j = 0; j < 16; ++j) sum += lanes[j];
    return sum;
}

static float dot_row(int32_t type, const uint8_t* row, const void* xq, size_t blocks) {
    switch (type) {
        case BRISK_TYPE_Q4_0: return dot_q4_0((const q4_0_t*)row, (const q8_0_t*)xq, blocks);
        case BRISK_TYPE_Q4_1: return dot_q4_1((const q4_1_t*)row, (const q8_0_t*)xq, blocks);
        case BRISK_TYPE_Q5_0: return dot_q5_0((const q5_0_t*)row, (const q8_0_t*)xq, blocks);
        case BRISK_TYPE_Q8_0: return dot_q8_0((const q8_0_t*)row, (const q8_0_t*)xq, blocks);
        case BRISK_TYPE_Q5_K: return dot_q5_k((const q5_k_t*)row, (const q8_k_t*)xq, blocks);
        case BRISK_TYPE_Q4_K: return dot_q4_k((const q4_k_t*)row, (const q8_k_t*)xq, blocks);
        case BRISK_TYPE_Q6_K: return dot_q6_k((const q6_k_t*)row, (const q8_k_t*)xq, blocks);
        default: return dot_tq2_0((const tq2_0_t*)row, (const q8_k_t*)xq, blocks);
    }
}

/* Session::multiply for one target (src/model.cpp:551-653) over generic matvec/matmul
 * (src/kernels.cpp:13-30): activations quantised per row once, out[t*rows + r] = dot(row r, x_t).
 * F32/F16 weights multiply raw f32 activations with dot_f32 (src/model.cpp:641-646; F16 tensors are
 * widened to f32 when the reference loads them, src/model.cpp:439-449, :526-528). */
typedef struct {
    int32_t type;
    const void* w;
    uint64_t rows, cols, n;
    const float* x;
    const uint8_t* xq;
    size_t blocks, bb, xb;
    float* out;
} mm_job;

static void mm_rows_float(void* p, int64_t r0, int64_t r1) {
    const mm_job* j = (const mm_job*)p;
    float* wide = (float*)malloc(j->cols * sizeof(float));
    for (int64_t r = r0; r < r1; ++r) {
        const float* wr;
        if (j->type == BRISK_TYPE_F32) {
            wr = (const float*)j->w + (size_t)r * j->cols;
        } else {
            const uint16_t* h = (const uint16_t*)j->w + (size_t)r * j->cols;
            for (size_t i = 0; i < j->cols; ++i) wide[i] = j->type == BRISK_TYPE_BF16 ? bfloat_to_float(h[i]) : oracle_half_to_float(h[i]);
            wr = wide;
        }
        for (uint64_t t = 0; t < j->n; ++t) j->out[t * j->rows + r] = dot_f32(wr, j->x + t * j->cols, j->cols);
    }
    free(wide);
}

static void mm_rows_quant(void* p, int64_t r0, int64_t r1) {
    const mm_job* j = (const mm_job*)p;
    for (int64_t r = r0; r < r1; ++r) {
        const uint8_t* row = (const uint8_t*)j->w + (size_t)r * j->blocks * j->bb;
        for (uint64_t t = 0; t < j->n; ++t) j->out[t * j->rows + r] = dot_row(j->type, row, j->xq + t * j->blocks * j->xb, j->blocks);
    }
}

int oracle_matmul(int32_t type, const void* w, uint64_t rows, uint64_t cols, const float* x, uint64_t n, float* out) {
    mm_job j = {type, w, rows, cols, n, x, NULL, 0, 0, 0, out};
    if (type_is_float(type)) {
        parallel_for((int64_t)rows, mm_rows_float, &j);
        return 0;
    }
    const size_t be = type_block_elems(type), bb = type_block_bytes(type);
    if (bb == 0 || be == 1 || cols % be != 0) return -1;
    const size_t blocks = cols / be;
    const int k = type_takes_q8_k(type);
    const size_t xb = k ? sizeof(q8_k_t) : sizeof(q8_0_t);
    uint8_t* xq = (uint8_t*)malloc(n * blocks * xb);
    if (!xq) return -1;
    for (uint64_t t = 0; t < n; ++t) {
        if (k) oracle_quantize_q8_k(x + t * cols, xq + t * blocks * xb, cols);
        else oracle_quantize_q8_0(x + t * cols, xq + t * blocks * xb, cols);
    }
    j.xq = xq;
    j.blocks = blocks;
    j.bb = bb;
    j.xb = xb;
    parallel_for((int64_t)rows, mm_rows_quant, &j);
    free(xq);
    return 0;
}

/* ---- the forward pass ---- */

struct oracle_session {
    brisk_cuda_model m;
    brisk_cuda_layer* layers;
    uint64_t max_context, position;
    uint16_t** keys;   /* per layer: [kv head][max_context][head_dim] f16 (src/model.cpp:982-991) */
    uint16_t** values;
    float *hidden, *normed, *query, *newk, *newv, *attended, *projected, *gate, *up, *rope, *rope_local, *logits, *trace;
};

#define MAXB 256 /* kMaxBatch, src/model.cpp:533 */

/* rms_norm, src/model.cpp:87-97: squares in f32, sum in double, scale = 1/sqrt(mean+eps) in f32. */
static void rms_norm(const float* x, const float* w, float eps, float* out, size_t n) {
    double sum = 0.0;
    for (size_t i = 0; i < n; ++i) sum += (double)(x[i] * x[i]);
    const float mean = (float)(sum / (double)n);
    const float scale = 1.0f / sqrtf(mean + eps);
    for (size_t i = 0; i < n; ++i) out[i] = x[i] * scale * w[i];
}

/* apply_rope, src/model.cpp:104-115 */
static void apply_rope(float* head, const float* rope, size_t dim, int neox) {
    const size_t half = dim / 2;
    for (size_t i = 0; i < half; ++i) {
        const float c = rope[2 * i], s = rope[2 * i + 1];
        float* a = &head[neox ? i : 2 * i];
        float* b = &head[neox ? i + half : 2 * i + 1];
        const float x0 = *a, x1 = *b;
        *a = x0 * c - x1 * s;
        *b = x0 * s + x1 * c;
    }
}

static void embedding_row(const brisk_cuda_matrix* e, size_t r, float* out) {
    const size_t row_bytes = e->cols / type_block_elems(e->type) * type_block_bytes(e->type);
    oracle_dequantize(e->type, (const uint8_t*)e->data + r * row_bytes, out, e->cols);
}

oracle_session* oracle_session_create(const brisk_cuda_model* model, uint64_t max_context) {
    oracle_session* s = (oracle_session*)calloc(1, sizeof(*s));
    s->m = *model;
    s->layers = (brisk_cuda_layer*)malloc(sizeof(brisk_cuda_layer) * model->layer_count);
    memcpy(s->layers, model->layers, sizeof(brisk_cuda_layer) * model->layer_count);
    s->m.layers = s->layers;
    s->max_context = max_context == 0 || max_context > model->context_length ? model->context_length : max_context;
    const size_t H = model->hidden, Q = (size_t)model->head_count * model->head_dim, KV = (size_t)model->kv_head_count * model->head_dim;
    s->keys = (uint16_t**)calloc(model->layer_count, sizeof(uint16_t*));
    s->values = (uint16_t**)calloc(model->layer_count, sizeof(uint16_t*));
    for (uint32_t l = 0; l < model->layer_count; ++l) {
        s->keys[l] = (uint16_t*)calloc(KV * s->max_context, 2);
        s->values[l] = (uint16_t*)calloc(KV * s->max_context, 2);
    }
    s->hidden = (float*)malloc(MAXB * H * 4);
    s->normed = (float*)malloc(MAXB * H * 4);
    s->query = (float*)malloc(MAXB * Q * 4);
    s->newk = (float*)malloc(MAXB * KV * 4);
    s->newv = (float*)malloc(MAXB * KV * 4);
    s->attended = (float*)malloc(MAXB * Q * 4);
    s->projected = (float*)malloc(MAXB * H * 4);
    s->gate = (float*)malloc(MAXB * (size_t)model->ffn * 4);
    s->up = (float*)malloc(MAXB * (size_t)model->ffn * 4);
    s->rope = (float*)malloc(MAXB * (size_t)model->head_dim * 4);
    s->rope_local = (float*)malloc(MAXB * (size_t)model->head_dim * 4);
    s->logits = (float*)malloc(64 * (size_t)model->vocab_size * 4);
    s->trace = (float*)calloc((size_t)model->layer_count * H, 4);
    return s;
}

void oracle_session_destroy(oracle_session* s) {
    if (!s) return;
    for (uint32_t l = 0; l < s->m.layer_count; ++l) {
        free(s->keys[l]);
        free(s->values[l]);
    }
    free(s->keys); free(s->values); free(s->hidden); free(s->normed); free(s->query); free(s->newk); free(s->newv);
    free(s->attended); free(s->projected); free(s->gate); free(s->up); free(s->rope); free(s->rope_local); free(s->logits);
    free(s->trace); free(s->layers); free(s);
}

static void mm(const brisk_cuda_matrix* w, const float* x, size_t n, float* out) {
    oracle_matmul(w->type, w->data, w->rows, w->cols, x, n, out);
}

typedef struct { struct oracle_session* s; uint32_t layer; size_t n; float scale; } attn_job;

/* Causal attention (src/model.cpp:1050-1093 over src/kernels_f32.cpp:256-284): per (token, head):
 * score = dot_f32(q, k)*scale; softmax with f32 exp and a double sum; out += p * v, position by position. */
static void attention_range(void* p, int64_t i0, int64_t i1) {
    const attn_job* j = (const attn_job*)p;
    struct oracle_session* s = j->s;
    const brisk_cuda_model* c = &s->m;
    const size_t D = c->head_dim, Q = (size_t)c->head_count * D, group = c->head_count / c->kv_head_count;
    const uint32_t l = j->layer;
    float* sc = (float*)malloc((s->position + j->n) * sizeof(float));
    float key[1024];
    for (int64_t idx = i0; idx < i1; ++idx) {
        const size_t t = (size_t)idx / c->head_count, h = (size_t)idx % c->head_count;
        const size_t visible = s->position + t + 1, kvh = h / group;
        const float* q = s->query + t * Q + h * D;
        /* A sliding layer sees only the last sliding_window positions (src/model.cpp:1084-1085). */
        const size_t start = s->layers[l].slides && visible > c->sliding_window ? visible - c->sliding_window : 0;
        for (size_t pp = start; pp < visible; ++pp) {
            const uint16_t* kr = s->keys[l] + (kvh * s->max_context + pp) * D;
            for (size_t i = 0; i < D; ++i) key[i] = oracle_half_to_float(kr[i]);
            sc[pp] = dot_f32(q, key, D) * j->scale;
        }
        float mx = sc[start];
        for (size_t pp = start + 1; pp < visible; ++pp) mx = sc[pp] > mx ? sc[pp] : mx;
        double sum = 0.0;
        for (size_t pp = start; pp < visible; ++pp) {
            sc[pp] = expf(sc[pp] - mx);
            sum += sc[pp];
        }
        const float inv = (float)(1.0 / sum);
        for (size_t pp = start; pp < visible; ++pp) sc[pp] *= inv;
        float* out = s->attended + t * Q + h * D;
        for (size_t i = 0; i < D; ++i) out[i] = 0.0f;
        for (size_t pp = start; pp < visible; ++pp) {
            const uint16_t* vr = s->values[l] + (kvh * s->max_context + pp) * D;
            const float wgt = sc[pp];
            for (size_t i = 0; i < D; ++i) out[i] += wgt * oracle_half_to_float(vr[i]);
        }
    }
    free(sc);
}

/* Session::eval_batch, src/model.cpp:867-1212, for the qwen3 / llama / bitnet / gemma3 layer shapes. */
static void eval_batch(oracle_session* s, const int32_t* tokens, size_t n, int all_logits) {
    const brisk_cuda_model* c = &s->m;
    const size_t H = c->hidden, D = c->head_dim, Q = (size_t)c->head_count * D, KV = (size_t)c->kv_head_count * D, F = c->ffn;
    const size_t group = c->head_count / c->kv_head_count;
    const float eps = c->rms_epsilon;
    const int bitnet = c->arch == BRISK_ARCH_BITNET;

    /* cos/sin by repeated multiplication from pos (src/model.cpp:880-892). */
    /* Phi rotates only the first rope_dim values of a head; the angles are built for that width (:893, :1024). */
    const size_t RD = c->rope_dim != 0 && c->rope_dim < D ? c->rope_dim : D;
    const float attn_factor = c->rope_attn_factor != 0.0f ? c->rope_attn_factor : 1.0f;
    const float theta_scale = powf(c->rope_base, -2.0f / (float)RD);
    const float rope_scale = c->rope_scale != 0.0f ? c->rope_scale : 1.0f;
    for (size_t t = 0; t < n; ++t) {
        float theta = (float)(s->position + t) * rope_scale;
        float* rope = s->rope + t * D;
        for (size_t i = 0; i < RD / 2; ++i) {
            const float angle = c->rope_factor_count ? theta / c->rope_factors[i] : theta;
            rope[2 * i] = cosf(angle) * attn_factor;
            rope[2 * i + 1] = sinf(angle) * attn_factor;
            theta *= theta_scale;
        }
    }
    if (c->sliding_window != 0) { /* the sliding layers' table: their own base, scale 1, no divisors (:894) */
        const float local_scale = powf(c->rope_base_local, -2.0f / (float)D);
        for (size_t t = 0; t < n; ++t) {
            float theta = (float)(s->position + t) * 1.0f;
            float* rope = s->rope_local + t * D;
            for (size_t i = 0; i < D / 2; ++i) {
                rope[2 * i] = cosf(theta) * 1.0f;
                rope[2 * i + 1] = sinf(theta) * 1.0f;
                theta *= local_scale;
            }
        }
    }
    for (size_t t = 0; t < n; ++t) { /* :896-902 */
        embedding_row(&c->token_embd, (size_t)tokens[t], s->hidden + t * H);
        if (c->embedding_scale != 0.0f && c->embedding_scale != 1.0f)
            for (size_t i = 0; i < H; ++i) s->hidden[t * H + i] *= c->embedding_scale;
    }

    const float attn_scale = 1.0f / sqrtf((float)D); /* :978 */
    for (uint32_t l = 0; l < c->layer_count; ++l) {
        const brisk_cuda_layer* L = &s->layers[l];
        for (size_t t = 0; t < n; ++t) rms_norm(s->hidden + t * H, L->attn_norm, eps, s->normed + t * H, H); /* :996-1001 */
        mm(&L->q, s->normed, n, s->query); /* :1013-1015 */
        mm(&L->k, s->normed, n, s->newk);
        mm(&L->v, s->normed, n, s->newv);
        for (size_t t = 0; t < n; ++t) { /* :1022-1046 */
            const int local = L->slides && c->sliding_window != 0;
            const float* rope = (local ? s->rope_local : s->rope) + t * D; /* :1024-1025 */
            const size_t W = local ? D : RD; /* rotated width */
            if (L->q_bias) { /* add_bias, :1026-1030 (src/model.cpp:117-119) */
                for (size_t i = 0; i < Q; ++i) s->query[t * Q + i] += L->q_bias[i];
                for (size_t i = 0; i < KV; ++i) s->newk[t * KV + i] += L->k_bias[i];
                for (size_t i = 0; i < KV; ++i) s->newv[t * KV + i] += L->v_bias[i];
            }
            for (size_t h = 0; h < c->head_count; ++h) {
                float* q = s->query + t * Q + h * D;
                if (L->q_norm) rms_norm(q, L->q_norm, eps, q, D);
                if (!L->no_rope) apply_rope(q, rope, W, c->rope_neox); /* rope_dim 0 on SmolLM3's NoPE layers, :1024 */
            }
            for (size_t h = 0; h < c->kv_head_count; ++h) {
                float* k = s->newk + t * KV + h * D;
                float* v = s->newv + t * KV + h * D;
                if (L->k_norm) rms_norm(k, L->k_norm, eps, k, D);
                if (!L->no_rope) apply_rope(k, rope, W, c->rope_neox);
                uint16_t* kc = s->keys[l] + (h * s->max_context + s->position + t) * D;
                uint16_t* vc = s->values[l] + (h * s->max_context + s->position + t) * D;
                for (size_t i = 0; i < D; ++i) {
                    kc[i] = oracle_float_to_half(k[i]);
                    vc[i] = oracle_float_to_half(v[i]);
                }
            }
        }
        {
            attn_job aj = {s, l, n, attn_scale};
            parallel_for((int64_t)(n * c->head_count), attention_range, &aj);
        }
        if (L->attn_sub_norm) /* :1095-1101 */
            for (size_t t = 0; t < n; ++t) rms_norm(s->attended + t * Q, L->attn_sub_norm, eps, s->attended + t * Q, Q);
        mm(&L->o, s->attended, n, s->projected); /* :1109 */
        for (size_t t = 0; t < n; ++t) {          /* :1111-1123 */
            float* h = s->hidden + t * H;
            float* p = s->projected + t * H;
            if (L->attn_post_norm) rms_norm(p, L->attn_post_norm, eps, p, H); /* Gemma, :1116-1119 */
            for (size_t i = 0; i < H; ++i) h[i] += p[i];
            rms_norm(h, L->ffn_norm, eps, s->normed + t * H, H);
        }
        mm(&L->gate, s->normed, n, s->gate); /* :1124-1127 */
        mm(&L->up, s->normed, n, s->up);
        for (size_t t = 0; t < n; ++t) { /* :1128-1149 */
            float* g = s->gate + t * F;
            const float* u = s->up + t * F;
            if (bitnet) {
                for (size_t i = 0; i < F; ++i) {
                    const float r = fmaxf(g[i], 0.0f);
                    g[i] = r * r * u[i];
                }
            } else if (c->gelu) { /* gelu_mul_f32, src/kernels_f32.cpp:291-296 */
                for (size_t i = 0; i < F; ++i) {
                    const float x = g[i];
                    g[i] = 0.5f * x * (1.0f + tanhf(0.7978845608f * (x + 0.044715f * x * x * x))) * u[i];
                }
            } else {
                for (size_t i = 0; i < F; ++i) g[i] = g[i] / (1.0f + expf(-g[i])) * u[i]; /* src/kernels_f32.cpp:287-289 */
            }
            if (L->ffn_sub_norm) rms_norm(g, L->ffn_sub_norm, eps, g, F);
        }
        mm(&L->down, s->gate, n, s->projected); /* :1150 */
        for (size_t t = 0; t < n; ++t) {         /* :1151-1162 */
            float* h = s->hidden + t * H;
            float* p = s->projected + t * H;
            if (L->ffn_post_norm) rms_norm(p, L->ffn_post_norm, eps, p, H); /* Gemma, :1155-1158 */
            for (size_t i = 0; i < H; ++i) h[i] += p[i];
        }
        memcpy(s->trace + (size_t)l * H, s->hidden + (n - 1) * H, H * 4);
    }
    const brisk_cuda_matrix* head = c->output.data ? &c->output : &c->token_embd; /* tied head, :328-330 */
    if (all_logits) { /* :1195-1200 */
        for (size_t t = 0; t < n; ++t) rms_norm(s->hidden + t * H, c->output_norm, eps, s->normed + t * H, H);
        mm(head, s->normed, n, s->logits);
    } else { /* :1201-1205 */
        rms_norm(s->hidden + (n - 1) * H, c->output_norm, eps, s->normed, H);
        mm(head, s->normed, 1, s->logits);
    }
    if (c->final_softcap != 0.0f) { /* :1206-1209 */
        const size_t count = (all_logits ? n : 1) * (size_t)c->vocab_size;
        for (size_t i = 0; i < count; ++i) s->logits[i] = c->final_softcap * tanhf(s->logits[i] / c->final_softcap);
    }
    s->position += n;
}

/* Session::eval / eval_all, src/model.cpp:704-727 */
int oracle_session_eval(oracle_session* s, const int32_t* tokens, uint64_t n, int all_logits, float* logits_out) {
    const uint32_t V = s->m.vocab_size;
    if (all_logits ? (n == 0 || n > 64) : n == 0) {
        set_error(all_logits ? "model: eval_all takes 1 to 64 tokens" : "model: no tokens to evaluate");
        return -1;
    }
    for (uint64_t i = 0; i < n; ++i)
        if (tokens[i] < 0 || (uint32_t)tokens[i] >= V) {
            set_error("model: token id out of range");
            return -1;
        }
    if (n > s->max_context - s->position) {
        set_error("model: context length exceeded");
        return -1;
    }
    if (all_logits) {
        eval_batch(s, tokens, n, 1);
        if (logits_out) memcpy(logits_out, s->logits, n * V * 4);
    } else {
        for (uint64_t b = 0; b < n; b += MAXB) eval_batch(s, tokens + b, n - b < MAXB ? n - b : MAXB, 0);
        if (logits_out) memcpy(logits_out, s->logits, (size_t)V * 4);
    }
    return 0;
}

/* Session::rollback, src/model.cpp:735-751 */
int oracle_session_rollback(oracle_session* s, uint64_t position) {
    if (position > s->position) {
        set_error("model: cannot roll forward");
        return -1;
    }
    s->position = position;
    return 0;
}

uint64_t oracle_session_position(const oracle_session* s) { return s->position; }

/* Scratch of the most recent batch, for layer-by-layer comparison with a one-layer model (the role of the
 * reference's BRISK_CPU_DEBUG dump, src/model.cpp:1183-1192). */
int oracle_session_debug_buffer(const oracle_session* s, const char* name, float* out, uint64_t count) {
    const float* b = !strcmp(name, "hidden") ? s->hidden : !strcmp(name, "query") ? s->query : !strcmp(name, "attended") ? s->attended
                     : !strcmp(name, "ffn") ? s->gate : !strcmp(name, "logits") ? s->logits : NULL;
    if (!b) return -1;
    memcpy(out, b, count * sizeof(float));
    return 0;
}

int oracle_session_layer_trace(const oracle_session* s, float* out) {
    memcpy(out, s->trace, (size_t)s->m.layer_count * s->m.hidden * 4);
    return 0;
}

/* Engine::log_likelihood, src/engine.cpp:10-33: chunks of 64 through eval_all; log-softmax in double. */
int oracle_session_log_likelihood(oracle_session* s, const int32_t* tokens, uint64_t n, double* out) {
    if (n < 2) {
        set_error("need at least two tokens to score");
        return -1;
    }
    const uint32_t V = s->m.vocab_size;
    double total = 0.0;
    for (uint64_t begin = 0; begin < n; begin += 64) {
        const uint64_t cnt = n - begin < 64 ? n - begin : 64;
        if (oracle_session_eval(s, tokens + begin, cnt, 1, NULL) != 0) return -1;
        for (uint64_t t = 0; t < cnt && begin + t + 1 < n; ++t) {
            const float* row = s->logits + t * V;
            float mx = row[0];
            for (uint32_t i = 1; i < V; ++i) mx = row[i] > mx ? row[i] : mx;
            double sum = 0.0;
            for (uint32_t i = 0; i < V; ++i) sum += exp((double)(row[i] - mx));
            total += (double)(row[tokens[begin + t + 1]] - mx) - log(sum);
        }
    }
    *out = total;
    return 0;
}

/* Greedy pick: first maximum (Sampler::sample with temperature <= 0, src/sampler.cpp:11-13). */
static int32_t argmax(const float* x, uint32_t n) {
    uint32_t best = 0;
    for (uint32_t i = 1; i < n; ++i)
        if (x[i] > x[best]) best = i;
    return (int32_t)best;
}

/* The generate loop, src/main.cpp:220-222, :288-299. */
int oracle_session_generate_greedy(oracle_session* s, const int32_t* prompt, uint64_t n_prompt, uint64_t steps,
                                   int32_t* out_tokens, float* out_logits) {
    const uint32_t V = s->m.vocab_size;
    if (oracle_session_eval(s, prompt, n_prompt, 0, NULL) != 0) return -1;
    for (uint64_t i = 0; i < steps; ++i) {
        if (out_logits) memcpy(out_logits + i * V, s->logits, (size_t)V * 4);
        const int32_t next = argmax(s->logits, V);
        out_tokens[i] = next;
        if (i + 1 < steps && oracle_session_eval(s, &next, 1, 0, NULL) != 0) return -1;
    }
    return 0;
}

/* LookupDrafter::draft, src/speculative.cpp:49-65: longest suffix (<= 3 tokens) with an earlier occurrence,
 * most recent occurrence first; copy what followed it. */
uint64_t oracle_lookup_draft(const int32_t* history, uint64_t n, uint64_t count, int32_t* out) {
    for (uint64_t ngram = n < 3 ? n : 3; ngram >= 1; --ngram) {
        const int32_t* suffix = history + n - ngram;
        for (uint64_t start = n - ngram; start-- > 0;) {
            if (memcmp(suffix, history + start, ngram * sizeof(int32_t)) == 0) {
                const uint64_t from = start + ngram;
                const uint64_t avail = count < n - from ? count : n - from;
                memcpy(out, history + from, avail * sizeof(int32_t));
                return avail;
            }
        }
    }
    return 0;
}

/* Speculator::step with a LookupDrafter, src/speculative.cpp:72-118, looped until `want` tokens are settled. */
int64_t oracle_session_speculate(oracle_session* s, const int32_t* prompt, uint64_t n_prompt, uint64_t draft_tokens,
                                 uint64_t want, int32_t* out, uint64_t* rounds, uint64_t* accepted_total) {
    const uint32_t V = s->m.vocab_size;
    if (draft_tokens > 63) draft_tokens = 63;
    uint64_t cap = n_prompt + want + 128, hn = n_prompt;
    int32_t* history = (int32_t*)malloc(cap * sizeof(int32_t));
    memcpy(history, prompt, n_prompt * sizeof(int32_t));
    if (n_prompt > 1 && oracle_session_eval(s, prompt, n_prompt - 1, 0, NULL) != 0) { free(history); return -1; }
    int32_t carry = prompt[n_prompt - 1];
    uint64_t written = 0, backoff = 0, last_backoff = 0, nrounds = 0, nacc = 0;
    int32_t batch[64], guesses[64], settled[64];
    while (written < want) {
        uint64_t ns = 0;
        if (backoff > 0) {
            --backoff;
            if (oracle_session_eval(s, &carry, 1, 0, NULL) != 0) { free(history); return -1; }
            settled[ns++] = argmax(s->logits, V);
        } else {
            const uint64_t ng = oracle_lookup_draft(history, hn, draft_tokens, guesses);
            const uint64_t base = s->position;
            batch[0] = carry;
            memcpy(batch + 1, guesses, ng * sizeof(int32_t));
            if (oracle_session_eval(s, batch, 1 + ng, 1, NULL) != 0) { free(history); return -1; }
            uint64_t acc = 0;
            int32_t next = argmax(s->logits, V);
            while (acc < ng && guesses[acc] == next) {
                settled[ns++] = next;
                ++acc;
                next = argmax(s->logits + acc * V, V);
            }
            settled[ns++] = next;
            oracle_session_rollback(s, base + 1 + acc);
            nacc += acc;
            if (acc == 0 && ng != 0) {
                last_backoff = last_backoff == 0 ? 1 : last_backoff * 2;
                if (last_backoff > 32) last_backoff = 32;
                backoff = last_backoff;
            } else {
                last_backoff /= 2;
            }
        }
        ++nrounds;
        if (hn + ns > cap) { cap = (hn + ns) * 2; history = (int32_t*)realloc(history, cap * sizeof(int32_t)); }
        memcpy(history + hn, settled, ns * sizeof(int32_t));
        hn += ns;
        carry = settled[ns - 1];
        for (uint64_t i = 0; i < ns && written < want; ++i) out[written++] = settled[i];
    }
    free(history);
    if (rounds) *rounds = nrounds;
    if (accepted_total) *accepted_total = nacc;
    return (int64_t)written;
}
