// extern "C" surface of the library (declared in include/poker2_b200.h).
#include "../../include/poker2_b200.h"

#include "common.cuh"

namespace p2b {
const char* last_error();
int launch_rank7_cards(const int16_t*, int64_t, int32_t*, cudaStream_t);
int launch_compare7_cards(const int16_t*, int64_t, int32_t*, cudaStream_t);
int launch_compare7_planes(const int8_t*, int64_t, int32_t*, cudaStream_t);
int launch_board_setup(const int16_t*, int64_t, unsigned char*, int32_t*, long long*, cudaStream_t);
int launch_showdown_eval(const unsigned char*, const int32_t*, const float*, int64_t, const long long*, const float*,
                         float*, int64_t, int64_t, cudaStream_t);
}  // namespace p2b

using namespace p2b;

#define P2B_REQUIRE(cond, msg) \
    do {                       \
        if (!(cond)) return set_error(P2B_ERR_ARG, "%s: %s", __func__, msg); \
    } while (0)

static_assert(P2B_TABLE_BYTES == 18592, "header and kernels disagree on the table size");

extern "C" {

const char* p2b_last_error(void) { return last_error(); }
int p2b_version(void) { return 1; }

int p2b_rank7_cards(const int16_t* cards, int64_t n, int32_t* out, void* stream) {
    P2B_REQUIRE(n >= 0, "negative count");
    P2B_REQUIRE(n == 0 || (cards && out), "null pointer");
    return launch_rank7_cards(cards, n, out, (cudaStream_t)stream);
}

int p2b_compare7_cards(const int16_t* cards, int64_t n, int32_t* out, void* stream) {
    P2B_REQUIRE(n >= 0, "negative count");
    P2B_REQUIRE(n == 0 || (cards && out), "null pointer");
    return launch_compare7_cards(cards, n, out, (cudaStream_t)stream);
}

int p2b_compare7_planes(const int8_t* planes, int64_t n, int32_t* out, void* stream) {
    P2B_REQUIRE(n >= 0, "negative count");
    P2B_REQUIRE(n == 0 || (planes && out), "null pointer");
    return launch_compare7_planes(planes, n, out, (cudaStream_t)stream);
}

int p2b_rank_hands(const int16_t* boards, int64_t m, int32_t* scores, int64_t* order, unsigned char* tables,
                   void* stream) {
    P2B_REQUIRE(m >= 0, "negative count");
    P2B_REQUIRE(m == 0 || boards, "null boards");
    P2B_REQUIRE(tables == nullptr || (reinterpret_cast<uintptr_t>(tables) & 15) == 0, "tables must be 16-byte aligned");
    return launch_board_setup(boards, m, tables, scores, reinterpret_cast<long long*>(order), (cudaStream_t)stream);
}

int p2b_showdown_values(const unsigned char* tables, const int32_t* table_of_row, const float* beliefs,
                        int64_t belief_row_stride, const int64_t* potential, const float* scale, float* values,
                        int64_t value_row_stride, int64_t rows, void* stream) {
    P2B_REQUIRE(rows >= 0, "negative count");
    P2B_REQUIRE(rows == 0 || (tables && beliefs && potential && scale && values), "null pointer");
    P2B_REQUIRE((reinterpret_cast<uintptr_t>(tables) & 15) == 0, "tables must be 16-byte aligned");
    P2B_REQUIRE(belief_row_stride >= 2 * P2B_NUM_HANDS && value_row_stride >= 2 * P2B_NUM_HANDS, "row stride too small");
    return launch_showdown_eval(tables, table_of_row, beliefs, belief_row_stride,
                                reinterpret_cast<const long long*>(potential), scale, values, value_row_stride, rows,
                                (cudaStream_t)stream);
}

}  // extern "C"
