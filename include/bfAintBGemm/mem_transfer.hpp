// Conversion of the fp32 master copies into device formats, host to host (interface of the reference's
// bfAintBGemm/mem_transfer.hpp:6-32: bf16 by truncation, int8 stored as value + 128), plus the formats the
// reference does not have: bf16 by round-to-nearest-even, two's-complement int8, packed int4.
#pragma once
#include <cstddef>
#include <cstdint>
#include "datatype.hpp"
#include "simple_device_mem.hpp"

template <typename Y, typename X, typename YLocation, typename XLocation>
void mem_transfer(YLocation& dst, XLocation& src, std::size_t size);

template <>
inline void mem_transfer<bfloat16, float, SimpleHostMem, SimpleHostMem>(SimpleHostMem& dst, SimpleHostMem& src, std::size_t size) {
    auto* out = static_cast<bfloat16*>(dst.GetBuffer());
    const auto* in = static_cast<const float*>(src.GetBuffer());
    for (std::size_t i = 0; i < size; ++i) out[i] = type_convert<bfloat16, float>(in[i]);
}
template <>
inline void mem_transfer<std::int8_t, float, SimpleHostMem, SimpleHostMem>(SimpleHostMem& dst, SimpleHostMem& src, std::size_t size) {
    auto* out = static_cast<std::uint8_t*>(dst.GetBuffer());
    const auto* in = static_cast<const float*>(src.GetBuffer());
    for (std::size_t i = 0; i < size; ++i) out[i] = static_cast<std::uint8_t>(type_convert<std::int8_t, float>(in[i]) + 128);  // offset-binary
}

// fp32 -> bf16 with round-to-nearest-even; when write_back is set the rounded value also replaces the fp32 master, so
// that the CPU check and the GPU see the same inputs (the reference feeds the unrounded master to its check,
// bfAintBGemm.cc:200-203, which is only right for values bf16 holds exactly).
inline void mem_transfer_bf16_rne(SimpleHostMem& dst, SimpleHostMem& src, std::size_t size, bool write_back = true) {
    auto* out = static_cast<bfloat16*>(dst.GetBuffer());
    auto* in = static_cast<float*>(src.GetBuffer());
    for (std::size_t i = 0; i < size; ++i) {
        out[i] = bf16_convert_rtn<bfloat16, float>(in[i]);
        if (write_back) in[i] = type_convert<float, bfloat16>(out[i]);
    }
}
inline void mem_transfer_int8_twos(SimpleHostMem& dst, SimpleHostMem& src, std::size_t size) {
    auto* out = static_cast<std::int8_t*>(dst.GetBuffer());
    const auto* in = static_cast<const float*>(src.GetBuffer());
    for (std::size_t i = 0; i < size; ++i) out[i] = static_cast<std::int8_t>(in[i]);
}
// Integers in [-8,7], two per byte, low nibble = even index; offset_binary stores value + 8.
inline void mem_transfer_int4(SimpleHostMem& dst, SimpleHostMem& src, std::size_t size, bool offset_binary) {
    auto* out = static_cast<std::uint8_t*>(dst.GetBuffer());
    const auto* in = static_cast<const float*>(src.GetBuffer());
    for (std::size_t i = 0; i < size; i += 2) {
        const int q0 = static_cast<int>(in[i]) + (offset_binary ? 8 : 0);
        const int q1 = (i + 1 < size ? static_cast<int>(in[i + 1]) : 0) + (offset_binary ? 8 : 0);
        out[i / 2] = static_cast<std::uint8_t>((q0 & 0xF) | ((q1 & 0xF) << 4));
    }
}
