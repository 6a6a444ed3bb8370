// Host-side numerics for the CPU transport and for test oracles: fp16 / bf16 conversion and the four
// reduction operators.  16-bit floats are combined in fp32 and rounded once (round-to-nearest-even),
// the same contract the device executor follows.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>
#include "common/base.h"

namespace hcclb {

inline float bf16_to_float(uint16_t v)
{
    uint32_t u = (uint32_t)v << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
inline uint16_t float_to_bf16(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);  // quiet NaN
    u += 0x7fffu + ((u >> 16) & 1);
    return (uint16_t)(u >> 16);
}
inline float fp16_to_float(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1f, man = h & 0x3ffu, u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else {
            int e = -1;
            do { ++e; man <<= 1; } while (!(man & 0x400u));
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) u = sign | 0x7f800000u | (man << 13);
    else u = sign | ((exp + 112) << 23) | (man << 13);
    float f;
    memcpy(&f, &u, 4);
    return f;
}
inline uint16_t float_to_fp16(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    uint32_t sign = (u >> 16) & 0x8000u, ax = u & 0x7fffffffu;
    if (ax >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (ax > 0x7f800000u ? 0x200u : 0));
    if (ax >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);  // overflow after rounding -> inf
    if (ax < 0x33000001u) return (uint16_t)sign;               // underflow to zero
    int e = (int)(ax >> 23) - 127;
    uint32_t man = (ax & 0x7fffffu) | 0x800000u;
    int shift = e < -14 ? (13 + (-14 - e)) : 13;
    uint32_t half_man = man >> shift, rem = man & ((1u << shift) - 1), halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half_man & 1))) ++half_man;
    uint32_t he = e < -14 ? 0 : (uint32_t)(e + 15);
    // half_man includes the implicit bit for normal numbers: adding it to the exponent field carries correctly
    uint32_t out = e < -14 ? half_man : ((he << 10) + (half_man - 0x400u));
    return (uint16_t)(sign | out);
}

template <class A>
inline A apply_op(int op, A x, A y)
{
    switch (op) {
        case HCCL_REDUCE_SUM: return (A)(x + y);
        case HCCL_REDUCE_PROD: return (A)(x * y);
        case HCCL_REDUCE_MAX: return x > y ? x : y;
        default: return x < y ? x : y;
    }
}

// Traits: storage type T, accumulation type Acc.
template <class T> struct NumPlain { using S = T; using Acc = T; static Acc ld(T v) { return v; } static T st(Acc v) { return v; } };
struct NumF16 { using S = uint16_t; using Acc = float; static float ld(uint16_t v) { return fp16_to_float(v); } static uint16_t st(float v) { return float_to_fp16(v); } };
struct NumBF16 { using S = uint16_t; using Acc = float; static float ld(uint16_t v) { return bf16_to_float(v); } static uint16_t st(float v) { return float_to_bf16(v); } };

// Calls f(Traits{}) for a reducible dtype; returns false for transport-only types.
template <class F>
inline bool dispatch_reduce_dtype(int dt, F &&f)
{
    switch (dt) {
        case HCCL_DATA_TYPE_INT8: f(NumPlain<int8_t>{}); return true;
        case HCCL_DATA_TYPE_UINT8: f(NumPlain<uint8_t>{}); return true;
        case HCCL_DATA_TYPE_INT16: f(NumPlain<int16_t>{}); return true;
        case HCCL_DATA_TYPE_UINT16: f(NumPlain<uint16_t>{}); return true;
        case HCCL_DATA_TYPE_INT32: f(NumPlain<int32_t>{}); return true;
        case HCCL_DATA_TYPE_UINT32: f(NumPlain<uint32_t>{}); return true;
        case HCCL_DATA_TYPE_INT64: f(NumPlain<int64_t>{}); return true;
        case HCCL_DATA_TYPE_UINT64: f(NumPlain<uint64_t>{}); return true;
        case HCCL_DATA_TYPE_FP32: f(NumPlain<float>{}); return true;
        case HCCL_DATA_TYPE_FP64: f(NumPlain<double>{}); return true;
        case HCCL_DATA_TYPE_FP16: f(NumF16{}); return true;
        case HCCL_DATA_TYPE_BFP16: f(NumBF16{}); return true;
        default: return false;
    }
}
inline bool dtype_reducible(int dt)
{
    return dispatch_reduce_dtype(dt, [](auto) {});
}

}  // namespace hcclb
