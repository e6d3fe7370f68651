// Instantiation helpers for the warp-specialised kernels: one switch over the vectors a thread
// owns, restricted at compile time to what the workload's register budget allows.
#pragma once

#include "ws_row_kernels.cuh"

namespace credit {

template <template <typename, int, int, bool> class Op, typename T, int W, int V>
const void* ws_entry(bool full) {
    return full ? (const void*)ws_row_kernel<Op<T, W, V, true>> : (const void*)ws_row_kernel<Op<T, W, V, false>>;
}

template <template <typename, int, int, bool> class Op, typename T, int W, int MAX_ELEMS>
const void* ws_pick(int vpt, bool full) {
    constexpr int E = 16 / static_cast<int>(sizeof(T));
    if constexpr (1 * E <= MAX_ELEMS) { if (vpt == 1) return ws_entry<Op, T, W, 1>(full); }
    if constexpr (2 * E <= MAX_ELEMS) { if (vpt == 2) return ws_entry<Op, T, W, 2>(full); }
    if constexpr (4 * E <= MAX_ELEMS) { if (vpt == 4) return ws_entry<Op, T, W, 4>(full); }
    if constexpr (8 * E <= MAX_ELEMS) { if (vpt == 8) return ws_entry<Op, T, W, 8>(full); }
    if constexpr (16 * E <= MAX_ELEMS) { if (vpt == 16) return ws_entry<Op, T, W, 16>(full); }
    return nullptr;
}

// out_warps 16 or 8; nullptr when the combination is not instantiated
template <template <typename, int, int, bool> class Op, typename T, bool BACKWARD>
const void* ws_pick_warps(int out_warps, int vpt, bool full) {
    if (out_warps == 16) return ws_pick<Op, T, 16, ws_max_elems_per_thread(BACKWARD, false)>(vpt, full);
    if (out_warps == 8) return ws_pick<Op, T, 8, ws_max_elems_per_thread(BACKWARD, true)>(vpt, full);
    return nullptr;
}

}  // namespace credit
