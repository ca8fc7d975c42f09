/*
 * poker2_b200 -- C ABI of the sm_100a subgame-solving kernels.
 *
 * Every entry point takes plain pointers and sizes.  Unless a parameter is marked
 * "host", pointers are DEVICE pointers of the current CUDA device, `stream` is a
 * cudaStream_t passed as void* (NULL = default stream), and the call only enqueues
 * work on that stream (no synchronisation, no allocation after the first call on a
 * device, which uploads two small constant tables).  Return value: 0 on success,
 * negative on error; p2b_last_error() then describes it (thread-local).
 *
 * The upstream project has no C interface: its boundary is a set of Python call
 * signatures.  Each declaration cites the upstream function whose work it does, by
 * path inside the upstream repository.
 */
#ifndef POKER2_B200_H
#define POKER2_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define P2B_NUM_HANDS 1326
#define P2B_TABLE_BYTES 18592 /* size of one per-board showdown table blob */

const char* p2b_last_error(void);
int p2b_version(void);

/* ---- hand ranking (src/p2/env/rules_triton.py) ---------------------------------- */

/* rank_7_cards_single_batch_triton (rules_triton.py:96-117): cards [n,7] int16 ids
 * 0..51 -> out [n] int32 packed score type<<20|k1<<16|..|k5. */
int p2b_rank7_cards(const int16_t* cards, int64_t n, int32_t* out, void* stream);

/* compare_7_cards_single_batch_triton (rules_triton.py:78-93): cards [n,2,7] int16 ->
 * out [n] int32 in {1,-1,0}. */
int p2b_compare7_cards(const int16_t* cards, int64_t n, int32_t* out, void* stream);

/* compare_7_single_batch_triton (rules_triton.py:36-51): planes [n,2,4,13] int8 one-hot
 * -> out [n] int32 in {1,-1,0}. */
int p2b_compare7_planes(const int8_t* planes, int64_t n, int32_t* out, void* stream);

/* rank_hands_triton (rules_triton.py:120-148): boards [m,5] int16 -> scores [m,1326]
 * int32 and order [m,1326] int64 (stable ascending argsort).  Either output may be
 * NULL.  `tables`, if not NULL, receives [m, P2B_TABLE_BYTES] showdown tables, the
 * counterpart of _init_hand_rank_data (src/p2/search/cfr_evaluator.py:406-482). */
int p2b_rank_hands(const int16_t* boards, int64_t m, int32_t* scores, int64_t* order,
                   unsigned char* tables, void* stream);

/* ---- showdown (src/p2/search/cfr_evaluator.py:484-601, _showdown_value_both) ------
 * beliefs/values: `rows` rows of [2,1326] fp32, consecutive rows `*_row_stride` floats
 * apart.  table_of_row [rows] int32 selects the table blob of each row (NULL = row i
 * uses blob i).  potential [rows,2] int64, scale [rows] fp32:
 * values[r,p,h] = EV_p(h | beliefs[r,1-p]) * potential[r,p] / scale[r]. */
int p2b_showdown_values(const unsigned char* tables, const int32_t* table_of_row,
                        const float* beliefs, int64_t belief_row_stride,
                        const int64_t* potential, const float* scale, float* values,
                        int64_t value_row_stride, int64_t rows, void* stream);

#ifdef __cplusplus
}
#endif
#endif
