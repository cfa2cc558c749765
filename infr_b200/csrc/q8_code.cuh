// One int8 code of the activation quantiser: `(v * id).round().clamp(-127.0, 127.0) as i8`
// (crates/infr-cpu/src/quant.rs:38, :71): round half away from zero; a NaN product gives 0 (what Rust's `as` makes of a
// NaN), an infinite one +-127.
#pragma once

namespace infr {

__device__ __forceinline__ int q8_round_code(float v, float id) {
    float x = v * id;
    x = x < -127.0f ? -127.0f : (x > 127.0f ? 127.0f : x);  // both comparisons are false for a NaN: it passes through
    const int t = __float2int_rz(x);                        // a NaN converts to 0
    const float fr = x - (float)t;                          // exact; a NaN stays one and fails both tests below
    return t + (fr >= 0.5f ? 1 : 0) - (fr <= -0.5f ? 1 : 0);
}

// The same without the clamp, for a FINITE id: with |v| <= amax and id = 1 / (amax / 127) the product stays below
// 127.5 in magnitude (two roundings of 2^-24 each), so rounding cannot leave [-127, 127].  (An infinite id - a block
// whose largest magnitude is so small that amax / 127 has a reciprocal beyond the largest float - needs the clamp.)
__device__ __forceinline__ int q8_round_code_inrange(float v, float id) {
    const float x = v * id;
    const int t = __float2int_rz(x);
    const float fr = x - (float)t;
    return t + (fr >= 0.5f ? 1 : 0) - (fr <= -0.5f ? 1 : 0);
}

// Four codes in one word, the first in the low byte (the codes are within [-127, 127]: the saturation never acts).
__device__ __forceinline__ uint32_t q8_pack4(int q0, int q1, int q2, int q3) {
    uint32_t hi, w;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(q3), "r"(q2));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(q1), "r"(q0), "r"(hi));
    return w;
}

// Sum of the four signed bytes of a word.
__device__ __forceinline__ int q8_sum4(uint32_t w) { return __dp4a((int)w, 0x01010101, 0); }

}  // namespace infr
