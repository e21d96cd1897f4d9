// Element types and scalar conversions of the host side.
// Mirrors the interface of the reference's bfAintBGemm/datatype.hpp (type aliases :4-7, type_convert :9-73,
// bf16_convert_rtn :76-121) so that host code written against it compiles unchanged; the bodies are written
// for a CUDA/C++17 host (no HIP header is needed: bf16 is carried as its 16-bit pattern).
#pragma once
#include <cstdint>
#include <cstring>
#include <type_traits>

using bfloat16 = unsigned short;  // bit pattern of a bf16 value
using bhalf_t = bfloat16;

namespace afb_detail {
inline std::uint32_t f32_bits(float f) { std::uint32_t u; std::memcpy(&u, &f, sizeof u); return u; }
inline float bits_f32(std::uint32_t u) { float f; std::memcpy(&f, &u, sizeof f); return f; }
}  // namespace afb_detail

// Generic conversion: a plain static_cast, const qualifiers stripped.
template <typename Y, typename X>
inline std::remove_const_t<Y> type_convert(X x) {
    static_assert(!std::is_reference_v<Y> && !std::is_reference_v<X>, "type_convert takes values");
    return static_cast<std::remove_const_t<Y>>(x);
}
// bf16 -> fp32: the pattern becomes the upper half of the float.
template <>
inline float type_convert<float, bhalf_t>(bhalf_t x) { return afb_detail::bits_f32(static_cast<std::uint32_t>(x) << 16); }
// fp32 -> bf16 by TRUNCATION (what the reference's mem_transfer and kernel epilogue do).
template <>
inline bhalf_t type_convert<bhalf_t, float>(float x) { return static_cast<bhalf_t>(afb_detail::f32_bits(x) >> 16); }
// bf16 <-> int8 through fp32.
template <>
inline std::int8_t type_convert<std::int8_t, bhalf_t>(bhalf_t x) { return static_cast<std::int8_t>(type_convert<float, bhalf_t>(x)); }
template <>
inline bhalf_t type_convert<bhalf_t, std::int8_t>(std::int8_t x) { return type_convert<bhalf_t, float>(static_cast<float>(x)); }

// fp32 -> bf16, round to nearest even; NaNs stay NaNs (a payload that lives only in the low half is kept alive by
// setting the lowest surviving mantissa bit).
template <typename Y, typename X>
Y bf16_convert_rtn(X x);
template <>
inline bhalf_t bf16_convert_rtn<bhalf_t, float>(float x) {
    std::uint32_t u = afb_detail::f32_bits(x);
    const bool finite = (u & 0x7f800000u) != 0x7f800000u;
    if (finite) u += 0x7fffu + ((u >> 16) & 1u);
    else if (u & 0xffffu) u |= 0x10000u;
    return static_cast<bhalf_t>(u >> 16);
}
