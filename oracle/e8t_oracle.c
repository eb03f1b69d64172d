/*
 * CPU oracle (C restatement) for the ternary-E8 quantized-linear path.
 *
 * TEST INFRASTRUCTURE ONLY: this file is the checker and the timed CPU
 * baseline; the shipped library never links or calls it.
 *
 * Parity status: PINNED against packed bytes / fp16 scales / fp32 decoded
 * weights produced by the live reference (fixtures under tests/golden/).
 *
 * Reference locations restated (paths inside the reference project):
 *   ojasx2/math/lattice.py:292-332   LUT order            -> e8t_build_tables
 *   ojasx2/math/lattice.py:338-384   pack                 -> e8t_oracle_encode
 *   ojasx2/math/lattice.py:386-419   unpack               -> e8t_oracle_decode
 *   ojasx2/math/csrc/ojasx_math_core.hpp:580-634  fused fwd -> e8t_oracle_linear
 *
 * Build: see the Makefile beside this file (-O2 -ffp-contract=off: the encoder
 * must not fuse multiply-adds, every product is rounded on its own).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>

#define E8T_POINTS 3281

static int8_t  g_coords[E8T_POINTS][8];
static int16_t g_raw_to_rank[6561];
static pthread_once_t g_once = PTHREAD_ONCE_INIT;

static void build_tables(void) {
    int rank = 0;
    for (int raw = 0; raw < 6561; ++raw) {
        int t = raw, sum = 0;
        int8_t d[8];
        for (int i = 0; i < 8; ++i) { d[i] = (int8_t)((t % 3) - 1); sum += d[i]; t /= 3; }
        g_raw_to_rank[raw] = 0;
        if (((sum % 2) + 2) % 2 == 0) {
            memcpy(g_coords[rank], d, 8);
            g_raw_to_rank[raw] = (int16_t)rank;
            ++rank;
        }
    }
}

void e8t_build_tables(void) { pthread_once(&g_once, build_tables); }

/* float -> IEEE binary16, round to nearest even (no hardware half needed). */
static uint16_t f32_to_f16(float f) {
    uint32_t x; memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t mant = x & 0x007FFFFFu;
    int32_t  exp  = (int32_t)((x >> 23) & 0xFF);
    if (exp == 0xFF) return (uint16_t)(sign | 0x7C00u | (mant ? 0x200u : 0));
    int32_t e = exp - 127 + 15;
    if (e >= 0x1F) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        mant |= 0x00800000u;
        uint32_t shift = (uint32_t)(14 - e);
        uint32_t half = mant >> shift;
        uint32_t rem = mant & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half & 1u))) ++half;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((uint32_t)e << 10) | (mant >> 13);
    uint32_t rem = mant & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) ++half;
    return (uint16_t)(sign | half);
}

static float f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1F, mant = h & 0x3FF, x;
    if (exp == 0) {
        if (mant == 0) x = sign;
        else {
            int e = -1;
            do { ++e; mant <<= 1; } while (!(mant & 0x400u));
            x = sign | ((uint32_t)(127 - 15 - e) << 23) | ((mant & 0x3FFu) << 13);
        }
    } else if (exp == 0x1F) x = sign | 0x7F800000u | (mant << 13);
    else x = sign | ((exp - 15 + 127) << 23) | (mant << 13);
    float f; memcpy(&f, &x, 4); return f;
}

/*
 * Encode `total` fp32 values (row-major flattened matrix, already widened from
 * fp16/bf16 if needed).  `group` must be a positive multiple of 16.  Outputs:
 * packed[ceil(total/group)*group*3/16], scales[ceil(total/group)] (binary16 bits).
 */
void e8t_oracle_encode(const float* w, int64_t total, int group,
                       uint8_t* packed, uint16_t* scales) {
    e8t_build_tables();
    const int64_t ngroups = (total + group - 1) / group;
    const float inv_div = (float)sqrt((double)group);   /* float(math.sqrt(g)) */
    float* buf = (float*)malloc(sizeof(float) * (size_t)group);
    int pending = -1;                                   /* first code of a pair */
    int64_t out = 0;
    for (int64_t gi = 0; gi < ngroups; ++gi) {
        for (int i = 0; i < group; ++i) {
            int64_t idx = gi * group + i;
            buf[i] = idx < total ? w[idx] : 0.0f;
        }
        /* eight lane accumulators, products rounded separately, lanes summed 0..7 */
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int d = 0; d < group; d += 8)
            for (int j = 0; j < 8; ++j) { float p = buf[d + j] * buf[d + j]; acc[j] = acc[j] + p; }
        float s = acc[0];
        for (int j = 1; j < 8; ++j) s = s + acc[j];
        float scale = sqrtf(s) / inv_div + 1e-8f;
        scales[gi] = f32_to_f16(scale);

        for (int b = 0; b < group; b += 8) {
            float v[8], q[8], alt[8], pen[8];
            int sum = 0;
            for (int i = 0; i < 8; ++i) {
                v[i] = buf[b + i] / scale;
                float r = rintf(v[i]);
                q[i] = r < -1.0f ? -1.0f : (r > 1.0f ? 1.0f : r);
                sum += (int)q[i];
                alt[i] = (q[i] == 0.0f) ? (v[i] >= 0.0f ? 1.0f : -1.0f) : 0.0f;
                float da = alt[i] - v[i], dq = q[i] - v[i];
                float da2 = da * da, dq2 = dq * dq;
                pen[i] = da2 - dq2;
            }
            if (((sum % 2) + 2) % 2 != 0) {
                int worst = 0;
                for (int i = 1; i < 8; ++i) if (pen[i] < pen[worst]) worst = i;
                q[worst] = alt[worst];
            }
            int raw = 0, p3 = 1;
            for (int i = 0; i < 8; ++i) { raw += ((int)q[i] + 1) * p3; p3 *= 3; }
            int code = g_raw_to_rank[raw];
            if (pending < 0) pending = code;
            else {
                packed[out + 0] = (uint8_t)(pending & 0xFF);
                packed[out + 1] = (uint8_t)(((pending >> 8) & 0x0F) | ((code & 0x0F) << 4));
                packed[out + 2] = (uint8_t)((code >> 4) & 0xFF);
                out += 3; pending = -1;
            }
        }
    }
    free(buf);
}

/* Decode `total` weights: W = float(coord) * float(scale_f16). */
void e8t_oracle_decode(const uint8_t* packed, const uint16_t* scales, int64_t total,
                       int group, float* out) {
    e8t_build_tables();
    for (int64_t base = 0; base < total; base += 16) {
        const uint8_t* t = packed + (base / 16) * 3;
        int c[2] = { t[0] | ((t[1] & 0x0F) << 8), ((t[1] >> 4) & 0x0F) | (t[2] << 4) };
        for (int h = 0; h < 2; ++h)
            for (int i = 0; i < 8; ++i) {
                int64_t idx = base + h * 8 + i;
                if (idx < total) out[idx] = (float)g_coords[c[h]][i] * f16_to_f32(scales[idx / group]);
            }
    }
}

/*
 * Fused forward with the accumulation order of the reference's native kernel:
 * per (m, n): acc = bias; per group: group_acc = sum x*coord (k ascending);
 * acc += group_acc * scale.  x, y fp32; rows of `packed` are K*3/16 bytes.
 */
void e8t_oracle_linear(const float* x, const uint8_t* packed, const uint16_t* scales,
                       const float* bias, float* y, int64_t M, int64_t K, int64_t N, int group) {
    e8t_build_tables();
    const int64_t row_bytes = K * 3 / 16, ngr = K / group, blocks = group / 16;
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            float acc = bias ? bias[n] : 0.0f;
            const uint8_t* wr = packed + n * row_bytes;
            const float* xr = x + m * K;
            for (int64_t g = 0; g < ngr; ++g) {
                float scale = f16_to_f32(scales[n * ngr + g]), ga = 0.0f;
                for (int64_t b = 0; b < blocks; ++b) {
                    const uint8_t* t = wr + (g * group * 3) / 16 + b * 3;
                    int c0 = t[0] | ((t[1] & 0x0F) << 8), c1 = ((t[1] >> 4) & 0x0F) | (t[2] << 4);
                    const float* xk = xr + g * group + b * 16;
                    for (int d = 0; d < 8; ++d) ga += xk[d] * (float)g_coords[c0][d];
                    for (int d = 0; d < 8; ++d) ga += xk[8 + d] * (float)g_coords[c1][d];
                }
                acc += ga * scale;
            }
            y[m * N + n] = acc;
        }
}

/* Multi-threaded wrapper over output rows n (CPU baseline timing only). */
typedef struct { const float* x; const uint8_t* p; const uint16_t* s; const float* b; float* y;
                 int64_t M, K, N, n0, n1; int group; } job_t;

static void* linear_job(void* arg) {
    job_t* j = (job_t*)arg;
    const int64_t row_bytes = j->K * 3 / 16, ngr = j->K / j->group;
    for (int64_t m = 0; m < j->M; ++m) {
        /* reuse the scalar kernel on a row slice: build a temporary y row */
        float* yrow = j->y + m * j->N;
        for (int64_t n = j->n0; n < j->n1; ++n) {
            float tmp;
            e8t_oracle_linear(j->x + m * j->K, j->p + n * row_bytes, j->s + n * ngr,
                              j->b ? j->b + n : NULL, &tmp, 1, j->K, 1, j->group);
            yrow[n] = tmp;
        }
    }
    return NULL;
}

void e8t_oracle_linear_mt(const float* x, const uint8_t* packed, const uint16_t* scales,
                          const float* bias, float* y, int64_t M, int64_t K, int64_t N,
                          int group, int threads) {
    e8t_build_tables();
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    pthread_t tid[256]; job_t jobs[256];
    for (int t = 0; t < threads; ++t) {
        jobs[t] = (job_t){ x, packed, scales, bias, y, M, K, N, N * t / threads, N * (t + 1) / threads, group };
        pthread_create(&tid[t], NULL, linear_job, &jobs[t]);
    }
    for (int t = 0; t < threads; ++t) pthread_join(tid[t], NULL);
}

/* Multi-threaded encode over whole groups (independent), for baseline timing. */
typedef struct { const float* w; int64_t total; int group; uint8_t* p; uint16_t* s; } ejob_t;
static void* encode_job(void* arg) {
    ejob_t* j = (ejob_t*)arg;
    e8t_oracle_encode(j->w, j->total, j->group, j->p, j->s);
    return NULL;
}
void e8t_oracle_encode_mt(const float* w, int64_t total, int group,
                          uint8_t* packed, uint16_t* scales, int threads) {
    e8t_build_tables();
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    int64_t ngroups = (total + group - 1) / group;
    pthread_t tid[256]; ejob_t jobs[256];
    int used = 0;
    for (int t = 0; t < threads; ++t) {
        int64_t g0 = ngroups * t / threads, g1 = ngroups * (t + 1) / threads;
        if (g1 <= g0) continue;
        int64_t e0 = g0 * group, e1 = g1 * group; if (e1 > total) e1 = total;
        jobs[used] = (ejob_t){ w + e0, e1 - e0, group, packed + e0 * 3 / 16, scales + g0 };
        pthread_create(&tid[used], NULL, encode_job, &jobs[used]);
        ++used;
    }
    for (int t = 0; t < used; ++t) pthread_join(tid[t], NULL);
}
