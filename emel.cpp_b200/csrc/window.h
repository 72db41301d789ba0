// What the Llama session needs of a layer streaming window (window.cu).
#pragma once

#include <cstdint>

struct emelb_ctx;
struct emelb_window;

namespace emelb {

bool window_streaming(const emelb_window* w);
emelb_ctx* window_ctx(const emelb_window* w);
int window_layer_count(const emelb_window* w);
// the slot offset of the extent of `layer` that starts at source address `host` and is `bytes` long
bool window_find_extent(const emelb_window* w, int layer, const void* host, uint64_t bytes, uint64_t* slot_offset);

}  // namespace emelb
