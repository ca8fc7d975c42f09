// Shared declarations of the sm_100a kernels: card/combo constants, error plumbing.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define P2B_NUM_HANDS 1326
#define P2B_NUM_CARDS 52
// Hand rows are padded to 1344 floats: every row of a [node][combo] array starts on a
// 16-byte boundary (128-bit loads and stores), and 672 threads x 2 hands (or 336 x 4) cover a
// row exactly, so the solver's row accesses need no bounds check.
#define P2B_HPAD 1344

namespace p2b {

// Records a message retrievable through p2b_last_error(); returns the code it is given.
int set_error(int code, const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);

// First combo index whose lower card is c (combos are the pairs c1<c2 in lexicographic
// order): off(c) = c*51 - c*(c-1)/2.
__host__ __device__ __forceinline__ int combo_row_offset(int c) { return c * 51 - (c * (c - 1)) / 2; }
// Index of the combo (a,b), a<b.
__host__ __device__ __forceinline__ int combo_index(int a, int b) { return combo_row_offset(a) + (b - a - 1); }

// Device table hand -> (c1,c2), filled once per device by ensure_tables().
struct ComboTable {
    uint8_t c1[P2B_NUM_HANDS];
    uint8_t c2[P2B_NUM_HANDS];
};
int ensure_tables();  // uploads the constant tables of the current device (idempotent)
const ComboTable* device_combo_table();
struct RankLut;
const RankLut* device_rank_lut();  // tables of the hand-ranking table walk (rank7.cuh)

}  // namespace p2b

// error codes of the C ABI
#define P2B_OK 0
#define P2B_ERR_ARG (-1)
#define P2B_ERR_CUDA (-2)
#define P2B_ERR_STATE (-3)
