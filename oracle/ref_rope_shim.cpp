// Shim that exposes the reference's own CPU RoPE (`rope_cpu`, a header-only template in the
// reference checkout, src/q_rope.h:3-35) through a C symbol.  TEST INFRASTRUCTURE ONLY.  The
// reference header is included from where it lies (-I<reference>/src at build time); nothing of it
// is copied into this repository.  Output goes to oracle/_ref/.
#include "q_rope.h"

extern "C" void ref_rope_cpu_f32(float* rotated_queries, const float* queries, const float* cosines,
                                 const float* sines, int F, int W, int Hq, int S, int E, int RotaryE) {
    rope_cpu<float>(rotated_queries, queries, cosines, sines, F, W, Hq, S, E, RotaryE);
}
