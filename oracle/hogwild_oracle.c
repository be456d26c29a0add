/*
 * Plain-C restatement of the Hogwild! attention op.  TEST INFRASTRUCTURE ONLY: it is compiled into
 * oracle/libhogwild_oracle.so and called by the tests as an independent checker (scalar loops, no
 * BLAS); the shipped library never links or calls it.
 *
 * Follows the reference's eager path:
 *   rotation  python/hogwild/attention.py:77-90  (and src/q_rope.h:3-35): rotate-half pairing,
 *             products rounded to fp32 separately, the sum rounded to the storage type
 *   attention python/hogwild/attention.py:38-67: per fragment fp32 q.k, key l hidden when
 *             l > locations[f,w,s], ONE softmax over the concatenation of all fragments, fp32 sum
 * Parity pin: checked against the reference's own outputs in tests/golden by tests/test_oracle.py.
 *
 * All tensors are passed as fp32 arrays holding values that are exactly representable in the
 * storage type `dtype` (0 = fp32, 1 = fp16, 2 = bf16); only the rotated query is rounded here.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static float round_bf16(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return x; /* NaN */
    u += 0x7fffu + ((u >> 16) & 1u);
    u &= 0xffff0000u;
    memcpy(&x, &u, 4);
    return x;
}

static float round_f16(float x) {
    /* round-to-nearest-even to 11 significant bits, with fp16 subnormals and overflow to inf */
    if (!isfinite(x) || x == 0.0f) return x;
    int e;
    float m = frexpf(fabsf(x), &e);               /* |x| = m * 2^e, m in [0.5, 1) */
    int bits = 11;
    if (e < -13) bits = 11 - (-13 - e);           /* subnormal range: exponent below 2^-14 */
    if (bits <= 0) {
        float tiny = ldexpf(1.0f, -24);
        float r = (fabsf(x) > tiny * 0.5f) ? tiny : 0.0f;
        return copysignf(r, x);
    }
    float scaled = ldexpf(m, bits);
    float r = nearbyintf(scaled);                 /* default rounding mode: nearest even */
    float y = ldexpf(r, e - bits);
    if (y > 65504.0f) y = INFINITY;
    return copysignf(y, x);
}

static float round_to(float x, int dtype) {
    return dtype == 2 ? round_bf16(x) : (dtype == 1 ? round_f16(x) : x);
}

/* rq[f,w,h,s,:] from q[w,h,s,:] and cos/sin[f,w,s,:]. */
void hogwild_rope_ref(float* rq, const float* q, const float* cs, const float* sn, int F, int W, int Hq, int S, int E,
                      int R, int dtype) {
    const int half = R / 2;
    for (int f = 0; f < F; ++f)
        for (int w = 0; w < W; ++w)
            for (int h = 0; h < Hq; ++h)
                for (int s = 0; s < S; ++s) {
                    const float* x = q + (((size_t)w * Hq + h) * S + s) * E;
                    const float* c = cs + (((size_t)f * W + w) * S + s) * R;
                    const float* t = sn + (((size_t)f * W + w) * S + s) * R;
                    float* y = rq + ((((size_t)f * W + w) * Hq + h) * S + s) * E;
                    for (int e = 0; e < half; ++e) {
                        volatile float a = x[e] * c[e], b = x[e + half] * t[e];
                        y[e] = round_to(a - b, dtype);
                        volatile float a2 = x[e + half] * c[e + half], b2 = x[e] * t[e + half];
                        y[e + half] = round_to(a2 + b2, dtype);
                    }
                    for (int e = R; e < E; ++e) y[e] = x[e];
                }
}

/*
 * out[w,hq,s,:] (fp32, not rounded).  rq [F,W,Hq,S,E]; keys[f] [Hkv,L_f,E]; values[f] [Hkv,L_f,Ev].
 * Rows that see no key are set to NaN, as the reference's softmax over nothing produces.
 */
void hogwild_sdpa_ref(float* out, const float* rq, const int32_t* loc, const float* const* keys,
                      const float* const* values, const int32_t* lens, float scale, int F, int W, int Hq, int Hkv, int S,
                      int E, int Ev) {
    const int G = Hq / Hkv;
    size_t total = 0;
    for (int f = 0; f < F; ++f) total += (size_t)lens[f];
    float* sc = (float*)malloc((total ? total : 1) * sizeof(float));
    for (int w = 0; w < W; ++w)
        for (int h = 0; h < Hq; ++h)
            for (int s = 0; s < S; ++s) {
                const int hk = h / G;
                size_t n = 0;
                float mx = -INFINITY;
                for (int f = 0; f < F; ++f) {
                    const float* qv = rq + ((((size_t)f * W + w) * Hq + h) * S + s) * E;
                    const int qpos = loc[((size_t)f * W + w) * S + s];
                    for (int l = 0; l < lens[f]; ++l, ++n) {
                        if (l > qpos) { sc[n] = -INFINITY; continue; }
                        const float* kv = keys[f] + ((size_t)hk * lens[f] + l) * E;
                        float acc = 0.f;
                        for (int e = 0; e < E; ++e) acc += qv[e] * kv[e];
                        sc[n] = scale * acc;
                        if (sc[n] > mx) mx = sc[n];
                    }
                }
                float* o = out + (((size_t)w * Hq + h) * S + s) * Ev;
                if (mx == -INFINITY) { for (int e = 0; e < Ev; ++e) o[e] = NAN; continue; }
                double den = 0.0;
                for (size_t i = 0; i < n; ++i) { sc[i] = expf(sc[i] - mx); den += sc[i]; }
                for (int e = 0; e < Ev; ++e) o[e] = 0.f;
                n = 0;
                for (int f = 0; f < F; ++f)
                    for (int l = 0; l < lens[f]; ++l, ++n) {
                        if (sc[n] == 0.f) continue;
                        const float p = (float)(sc[n] / den);
                        const float* vv = values[f] + ((size_t)hk * lens[f] + l) * Ev;
                        for (int e = 0; e < Ev; ++e) o[e] += p * vv[e];
                    }
            }
    free(sc);
}
