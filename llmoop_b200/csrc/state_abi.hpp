// Byte layouts of the reference's kernel ABI that a host may still want to
// exchange with reference tooling: the 20-byte stream-control record
// (runtime-rs/src/vulkan_stream_circuit/stream_control_bytes.rs:8-18) and the
// transient-state buffer header + page table
// (runtime-rs/src/vulkan_stream_circuit/transient_state_buffer_layout.rs:24-154).
// The CUDA backend itself addresses KV through a per-stream block table shared
// by all layers; these helpers let state dumps be compared with the reference's.
#pragma once

#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <vector>

namespace nerve {

inline void stream_control_bytes(uint32_t token, uint64_t tick, uint32_t flags, uint32_t capacity, uint8_t out[20]) {
    const uint32_t words[5] = {token, static_cast<uint32_t>(tick), static_cast<uint32_t>(tick >> 32), flags, capacity};
    std::memcpy(out, words, 20);
}

struct StateLayout {
    int64_t block_activation_capacity = 0, page_count = 0, page_bytes = 0, page_table_bytes = 0;
    int64_t static_offset = 0, dynamic_offset = 0, byte_capacity = 0, dynamic_capacity = 0, static_bytes = 0;
};

inline StateLayout state_layout(int64_t static_bytes, int64_t bytes_per_activation, int64_t max_dynamic, int64_t capacity) {
    constexpr int64_t kWindow = 64, kAlign = 256, kHeaderWords = 9;
    StateLayout layout;
    layout.static_bytes = static_bytes;
    if (bytes_per_activation > 0) {
        if (capacity == 0) throw std::runtime_error("state requires non-zero dynamic state capacity");
        layout.dynamic_capacity = max_dynamic > 0 && max_dynamic < capacity ? max_dynamic : capacity;
        layout.block_activation_capacity = layout.dynamic_capacity < kWindow ? layout.dynamic_capacity : kWindow;
        layout.page_bytes = bytes_per_activation * layout.block_activation_capacity;
        layout.page_count = (layout.dynamic_capacity + layout.block_activation_capacity - 1) / layout.block_activation_capacity;
    }
    if (static_bytes == 0 && layout.page_count == 0) throw std::runtime_error("state has unknown or zero byte capacity");
    layout.page_table_bytes = ((kHeaderWords + layout.page_count) * 4 + kAlign - 1) / kAlign * kAlign;
    layout.static_offset = layout.page_table_bytes;
    layout.dynamic_offset = (layout.static_offset + static_bytes + kAlign - 1) / kAlign * kAlign;
    layout.byte_capacity = layout.dynamic_offset + layout.page_bytes * layout.page_count;
    return layout;
}

// Header + page table with an explicit logical -> physical mapping (empty = identity).
inline std::vector<uint8_t> state_page_table_bytes(const StateLayout &layout, const std::vector<uint32_t> &mapping) {
    if (!mapping.empty() && static_cast<int64_t>(mapping.size()) != layout.page_count)
        throw std::runtime_error("transient page mapping has " + std::to_string(mapping.size()) + " entries but layout requires " +
                                 std::to_string(layout.page_count));
    std::vector<uint8_t> bytes(static_cast<size_t>(layout.page_table_bytes), 0);
    const uint32_t header[9] = {0x4e525653u,
                                1u,
                                static_cast<uint32_t>(layout.static_bytes),
                                static_cast<uint32_t>(layout.static_offset),
                                static_cast<uint32_t>(layout.page_bytes),
                                static_cast<uint32_t>(layout.page_count),
                                static_cast<uint32_t>(layout.dynamic_capacity),
                                static_cast<uint32_t>(layout.block_activation_capacity),
                                static_cast<uint32_t>(layout.dynamic_offset)};
    std::memcpy(bytes.data(), header, sizeof(header));
    for (int64_t page = 0; page < layout.page_count; page++) {
        uint32_t physical = mapping.empty() ? static_cast<uint32_t>(page) : mapping[static_cast<size_t>(page)];
        if (physical >= static_cast<uint32_t>(layout.page_count))
            throw std::runtime_error("transient physical page " + std::to_string(physical) + " exceeds capacity " +
                                     std::to_string(layout.page_count));
        std::memcpy(bytes.data() + (9 + page) * 4, &physical, 4);
    }
    return bytes;
}

// Tensor-parallel shard of `total` rows (or columns) that must stay in whole units (a head, 16 rows, a group of 128
// columns): rank r of `size` holds [begin, begin + count).  Throws when total is not a multiple of unit * size.
inline void tp_shard_range(int64_t total, int64_t unit, int rank, int size, int64_t &begin, int64_t &count) {
    if (size < 1 || rank < 0 || rank >= size || unit < 1) throw std::runtime_error("tensor-parallel rank/size/unit out of range");
    if (total % (unit * size) != 0)
        throw std::runtime_error(std::to_string(total) + " is not a multiple of " + std::to_string(unit) + " x " + std::to_string(size) + " ranks");
    count = total / size;
    begin = count * rank;
}

}  // namespace nerve
