// extern "C" surface of the library (declared in include/poker2_b200.h).
#include "../../include/poker2_b200.h"

#include "cfr.cuh"
#include "common.cuh"

namespace p2b {
const char* last_error();
int launch_rank7_cards(const int16_t*, int64_t, int32_t*, cudaStream_t);
int launch_compare7_cards(const int16_t*, int64_t, int32_t*, cudaStream_t);
int launch_compare7_planes(const int8_t*, int64_t, int32_t*, cudaStream_t);
int launch_board_setup(const int16_t*, int64_t, unsigned char*, int32_t*, long long*, cudaStream_t);
int launch_showdown_eval(const unsigned char*, const int32_t*, const float*, int64_t, const long long*, const float*,
                         float*, int64_t, int64_t, cudaStream_t);
int launch_showdown_ev_sorted(const float*, const int32_t*, const int32_t*, const int32_t*, const int32_t*, int64_t, int,
                              float, float*, cudaStream_t);
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

int p2b_showdown_ev_sorted(const float* b_sorted, const int32_t* c1_sorted, const int32_t* c2_sorted, const int32_t* l_idx,
                           const int32_t* r_idx, int64_t rows, int32_t hands, float eps, float* out, void* stream) {
    P2B_REQUIRE(rows >= 0 && hands >= 0, "negative count");
    P2B_REQUIRE(rows == 0 || hands == 0 || (b_sorted && c1_sorted && c2_sorted && l_idx && r_idx && out), "null pointer");
    return launch_showdown_ev_sorted(b_sorted, c1_sorted, c2_sorted, l_idx, r_idx, rows, hands, eps, out,
                                     (cudaStream_t)stream);
}

int p2b_cfr_default_blocks(void) { return cfr_default_blocks(); }

int p2b_cfr_path_policy(int32_t policy) { return cfr_path_policy(policy); }

int p2b_cfr_iteration_timing(int32_t enable) { return cfr_iteration_timing(enable); }

int p2b_cfr_iteration_ms(float* ms) {
    P2B_REQUIRE(ms != nullptr, "null pointer");
    return cfr_iteration_ms(ms);
}

int64_t p2b_cfr_scratch_floats(int32_t max_internal, int32_t num_blocks) {
    if (num_blocks <= 0) num_blocks = cfr_default_blocks();
    return cfr_scratch_floats(max_internal) * num_blocks;
}

int64_t p2b_cfr_solve_scratch_floats(int32_t max_internal, int32_t max_children, int32_t num_blocks,
                                     int32_t num_subgames, int64_t rows) {
    if (num_blocks <= 0) num_blocks = cfr_default_blocks();
    if (num_blocks > num_subgames) num_blocks = num_subgames > 0 ? num_subgames : 1;
    return cfr_solve_scratch_floats(max_internal, max_children, num_blocks, num_subgames, rows);
}

int p2b_cfr_solve(const void* subgames, const void* nodes, int32_t num_subgames, int64_t rows, int32_t max_children,
                  int32_t max_internal, const unsigned char* tables, const float* root_beliefs, float* regrets,
                  float* weight_sums, float* policy_avg, float* policy, float* root_values, float* values_avg,
                  float* beliefs_avg, float* exploitability, float* br_values, float* scratch, int64_t scratch_floats,
                  const void* scalars, int32_t iterations, int32_t flags, int32_t init_depth, int32_t* work_counter,
                  int32_t num_blocks, const int32_t* sample_pass, float* policy_sample, float* beliefs_last,
                  const int32_t* queue_order, const float* start_policy, float warm_start_weight, void* stream) {
    P2B_REQUIRE(num_subgames >= 0 && iterations >= 0 && rows >= 0, "negative count");
    P2B_REQUIRE(warm_start_weight >= 0.0f && (warm_start_weight == 0.0f || (start_policy && rows > 0)),
                "a warm start needs a start policy, the row count and a non-negative weight");
    P2B_REQUIRE((reinterpret_cast<uintptr_t>(start_policy) & 15) == 0, "all arrays must be 16-byte aligned");
    P2B_REQUIRE(!policy_sample || sample_pass, "policy_sample needs sample_pass");
    P2B_REQUIRE(((reinterpret_cast<uintptr_t>(policy_sample) | reinterpret_cast<uintptr_t>(beliefs_last)) & 15) == 0,
                "all arrays must be 16-byte aligned");
    if (num_subgames == 0) return P2B_OK;
    P2B_REQUIRE(subgames && nodes && root_beliefs && regrets && policy_avg && root_values && scratch && work_counter,
                "null pointer");
    P2B_REQUIRE(iterations == 0 || scalars, "null scalars");
    P2B_REQUIRE(max_internal >= 1, "max_internal must be positive");
    P2B_REQUIRE(!exploitability || values_avg, "exploitability needs values_avg");
    P2B_REQUIRE(flags >= 0 && flags <= 31 && !(flags & 8),
                "flags: bit 0 = CFR+ clamp, bit 1 = zero-sum value outputs, bit 2 = leaf values and regret weights at the "
                "average-policy beliefs, bit 4 = linear CFR");
    if (num_blocks <= 0) num_blocks = cfr_default_blocks();
    if (num_blocks > num_subgames) num_blocks = num_subgames;
    P2B_REQUIRE(scratch_floats >= cfr_scratch_floats(max_internal) * num_blocks, "scratch too small");
    const uintptr_t align = reinterpret_cast<uintptr_t>(subgames) | reinterpret_cast<uintptr_t>(nodes) |
                            reinterpret_cast<uintptr_t>(tables) | reinterpret_cast<uintptr_t>(root_beliefs) |
                            reinterpret_cast<uintptr_t>(regrets) | reinterpret_cast<uintptr_t>(weight_sums) |
                            reinterpret_cast<uintptr_t>(policy_avg) | reinterpret_cast<uintptr_t>(policy) |
                            reinterpret_cast<uintptr_t>(root_values) | reinterpret_cast<uintptr_t>(values_avg) |
                            reinterpret_cast<uintptr_t>(beliefs_avg) | reinterpret_cast<uintptr_t>(scratch);
    P2B_REQUIRE((align & 15) == 0, "all arrays must be 16-byte aligned");
    CfrParams p{};
    p.subgames = static_cast<const SubgameRec*>(subgames);
    p.nodes = static_cast<const NodeRecPacked*>(nodes);
    p.num_subgames = num_subgames;
    p.tables = tables;
    p.root_beliefs = root_beliefs;
    p.regrets = regrets;
    p.weight_sums = weight_sums;
    p.policy_avg = policy_avg;
    p.policy = policy;
    p.root_values = root_values;
    p.values_avg = values_avg;
    p.beliefs_avg = beliefs_avg;
    p.exploitability = exploitability;
    p.br_values = br_values;
    p.scratch = scratch;
    p.scratch_stride = cfr_scratch_floats(max_internal);
    p.max_internal = max_internal;
    p.scalars = static_cast<const IterScalars*>(scalars);
    p.iterations = iterations;
    p.cfr_plus = flags & 1;
    p.enforce_zero_sum = (flags >> 1) & 1;
    p.cfr_avg = (flags >> 2) & 1;
    p.linear = (flags >> 4) & 1;
    p.init_depth = init_depth;
    p.work_counter = work_counter;
    p.sample_pass = sample_pass;
    p.policy_sample = policy_sample;
    p.beliefs_last = beliefs_last;
    p.rows = rows;
    p.queue_order = queue_order;
    p.start_policy = start_policy;
    p.warm_weight = warm_start_weight;
    // with the larger scratch area of p2b_cfr_solve_scratch_floats the iteration passes of a plain
    // solve run in the lean iteration kernel
    const bool fast_scratch =
        scratch_floats >= cfr_solve_scratch_floats(max_internal, max_children, num_blocks, num_subgames, rows);
    return launch_cfr_solve(p, num_blocks, max_children, (cudaStream_t)stream, fast_scratch);
}

// Part of a solve: the passes pass_begin..pass_end, top-down and/or bottom-up sweeps.
int p2b_cfr_step(const void* subgames, const void* nodes, int32_t num_subgames, int64_t rows, int32_t max_children,
                 int32_t max_internal, const unsigned char* tables, const float* root_beliefs, float* regrets,
                 float* weight_sums, float* policy_avg, float* policy, float* root_values, float* values_avg,
                 float* beliefs_avg, float* exploitability, float* br_values, float* scratch, int64_t scratch_floats,
                 const void* scalars, int32_t iterations, int32_t flags, int32_t init_depth, int32_t* work_counter,
                 int32_t num_blocks, int32_t pass_begin, int32_t pass_end, int32_t phases, float* carry_sums,
                 float* carry_roots, const int32_t* leaf_begin, int32_t leaf_slots, float* leaf_beliefs,
                 const float* leaf_values, const int32_t* sample_pass, float* policy_sample, float* beliefs_last,
                 const int32_t* queue_order, const float* start_policy, void* stream) {
    P2B_REQUIRE(num_subgames >= 0 && iterations >= 1 && rows >= 0 && leaf_slots >= 0, "bad count");
    P2B_REQUIRE((reinterpret_cast<uintptr_t>(start_policy) & 15) == 0, "all row arrays must be 16-byte aligned");
    P2B_REQUIRE(!policy_sample || sample_pass, "policy_sample needs sample_pass");
    P2B_REQUIRE(((reinterpret_cast<uintptr_t>(policy_sample) | reinterpret_cast<uintptr_t>(beliefs_last)) & 15) == 0,
                "all row arrays must be 16-byte aligned");
    if (num_subgames == 0) return P2B_OK;
    P2B_REQUIRE(subgames && nodes && root_beliefs && regrets && policy_avg && root_values && scratch && work_counter &&
                    scalars && carry_sums && carry_roots,
                "null pointer");
    P2B_REQUIRE(max_internal >= 1, "max_internal must be positive");
    P2B_REQUIRE(!exploitability || values_avg, "exploitability needs values_avg");
    P2B_REQUIRE(flags >= 0 && flags <= 31,
                "flags: bit 0 = CFR+ clamp, bit 1 = zero-sum value outputs, bit 2 = leaf values and regret weights at the "
                "average-policy beliefs, bit 3 = keep the node values of every pass, bit 4 = linear CFR");
    P2B_REQUIRE(!(flags & 8) || (values_avg && beliefs_avg), "flags bit 3 needs values_avg and beliefs_avg");
    P2B_REQUIRE(pass_begin >= -1 && pass_begin <= pass_end && pass_end <= iterations, "pass range outside [-1, iterations]");
    P2B_REQUIRE((phases >= 1 && phases <= 3) || phases == 4 || phases == 8 || phases == 16,
                "phases must be 1 (top-down), 2 (bottom-up), 3 (both), 4 (best responses only), 8 (best-response pass of "
                "a warm start) or 16 (bottom-up sweep of pass_begin, then top-down sweep of pass_begin + 1)");
    P2B_REQUIRE(phases != 8 || (pass_begin == -1 && values_avg), "phases = 8 runs after the start pass and needs values_avg");
    P2B_REQUIRE(phases == 3 || phases == 16 || pass_begin == pass_end, "a single sweep direction covers exactly one pass");
    P2B_REQUIRE(phases != 16 || pass_end == pass_begin + 1, "phases = 16 joins two consecutive passes");
    P2B_REQUIRE(phases != 4 || (pass_begin == iterations && exploitability), "phases = 4 runs after the final pass and needs "
                                                                              "the exploitability output");
    P2B_REQUIRE((!leaf_beliefs && !leaf_values) || leaf_begin, "leaf arrays need leaf_begin");
    if (num_blocks <= 0) num_blocks = cfr_default_blocks();
    if (num_blocks > num_subgames) num_blocks = num_subgames;
    P2B_REQUIRE(scratch_floats >= cfr_scratch_floats(max_internal) * num_subgames,
                "scratch too small (stepped solves keep one set of work rows per subgame)");
    const uintptr_t align = reinterpret_cast<uintptr_t>(subgames) | reinterpret_cast<uintptr_t>(nodes) |
                            reinterpret_cast<uintptr_t>(tables) | reinterpret_cast<uintptr_t>(root_beliefs) |
                            reinterpret_cast<uintptr_t>(regrets) | reinterpret_cast<uintptr_t>(weight_sums) |
                            reinterpret_cast<uintptr_t>(policy_avg) | reinterpret_cast<uintptr_t>(policy) |
                            reinterpret_cast<uintptr_t>(root_values) | reinterpret_cast<uintptr_t>(values_avg) |
                            reinterpret_cast<uintptr_t>(beliefs_avg) | reinterpret_cast<uintptr_t>(scratch) |
                            reinterpret_cast<uintptr_t>(carry_roots) | reinterpret_cast<uintptr_t>(leaf_beliefs) |
                            reinterpret_cast<uintptr_t>(leaf_values);
    P2B_REQUIRE((align & 15) == 0, "all row arrays must be 16-byte aligned");
    CfrParams p{};
    p.subgames = static_cast<const SubgameRec*>(subgames);
    p.nodes = static_cast<const NodeRecPacked*>(nodes);
    p.num_subgames = num_subgames;
    p.tables = tables;
    p.root_beliefs = root_beliefs;
    p.regrets = regrets;
    p.weight_sums = weight_sums;
    p.policy_avg = policy_avg;
    p.policy = policy;
    p.root_values = root_values;
    p.values_avg = values_avg;
    p.beliefs_avg = beliefs_avg;
    p.exploitability = exploitability;
    p.br_values = br_values;
    p.scratch = scratch;
    p.scratch_stride = cfr_scratch_floats(max_internal);
    p.max_internal = max_internal;
    p.scalars = static_cast<const IterScalars*>(scalars);
    p.iterations = iterations;
    p.cfr_plus = flags & 1;
    p.enforce_zero_sum = (flags >> 1) & 1;
    p.cfr_avg = (flags >> 2) & 1;
    p.linear = (flags >> 4) & 1;
    p.iter_values = (flags >> 3) & 1;
    p.init_depth = init_depth;
    p.work_counter = work_counter;
    p.stepped = 1;
    p.pass_begin = pass_begin;
    p.pass_end = pass_end;
    p.phases = phases;
    p.carry_sums = carry_sums;
    p.carry_roots = carry_roots;
    p.leaf_begin = leaf_begin;
    p.leaf_beliefs = leaf_beliefs;
    p.leaf_values = leaf_values;
    p.sample_pass = sample_pass;
    p.policy_sample = policy_sample;
    p.beliefs_last = beliefs_last;
    p.queue_order = queue_order;
    p.start_policy = start_policy;
    p.rows = rows;
    p.leaf_slots = leaf_slots;
    return launch_cfr_solve(p, num_blocks, max_children, (cudaStream_t)stream);
}

int p2b_cfr_warm_seed(const void* nodes, int64_t rows, const float* start_policy, float weight, float* regrets,
                      float* weight_sums, void* stream) {
    P2B_REQUIRE(rows >= 0, "negative count");
    if (rows == 0) return P2B_OK;
    P2B_REQUIRE(nodes && start_policy && regrets, "null pointer");
    P2B_REQUIRE(weight > 0.0f, "the weight must be positive");
    return launch_cfr_warm_seed(static_cast<const NodeRecPacked*>(nodes), rows, start_policy, weight, regrets, weight_sums,
                                (cudaStream_t)stream);
}

int64_t p2b_cfr_noalloc_scratch_floats(void) { return cfr_static_scratch_floats(); }

// Allocation-free twin of p2b_cfr_solve: work rows, queue counter and combo table come from
// a fixed device area inside the library (see launch_cfr_solve_static).
int p2b_cfr_noalloc_status(int32_t* status, void* stream) {
    P2B_REQUIRE(status != nullptr, "null pointer");
    return cfr_static_status(status, (cudaStream_t)stream);
}

int p2b_cfr_solve_noalloc(const void* subgames, const void* nodes, int32_t num_subgames, int64_t rows,
                          int32_t max_children, int32_t max_internal, const unsigned char* tables, const float* root_beliefs, float* regrets,
                          float* weight_sums, float* policy_avg, float* policy, float* root_values, float* values_avg,
                          float* beliefs_avg, float* exploitability, float* br_values, const void* scalars,
                          int32_t iterations, int32_t flags, int32_t init_depth, void* stream) {
    P2B_REQUIRE(num_subgames >= 0 && iterations >= 0 && rows >= 0, "negative count");
    if (num_subgames == 0) return P2B_OK;
    P2B_REQUIRE(subgames && nodes && root_beliefs && regrets && policy_avg && root_values && scalars, "null pointer");
    P2B_REQUIRE(max_internal >= 1, "max_internal must be positive");
    P2B_REQUIRE(!exploitability || values_avg, "exploitability needs values_avg");
    P2B_REQUIRE(flags >= 0 && flags <= 31 && !(flags & 8),
                "flags: bit 0 = CFR+ clamp, bit 1 = zero-sum value outputs, bit 2 = leaf values and regret weights at the "
                "average-policy beliefs, bit 4 = linear CFR");
    const uintptr_t align = reinterpret_cast<uintptr_t>(subgames) | reinterpret_cast<uintptr_t>(nodes) |
                            reinterpret_cast<uintptr_t>(tables) | reinterpret_cast<uintptr_t>(root_beliefs) |
                            reinterpret_cast<uintptr_t>(regrets) | reinterpret_cast<uintptr_t>(weight_sums) |
                            reinterpret_cast<uintptr_t>(policy_avg) | reinterpret_cast<uintptr_t>(policy) |
                            reinterpret_cast<uintptr_t>(root_values) | reinterpret_cast<uintptr_t>(values_avg) |
                            reinterpret_cast<uintptr_t>(beliefs_avg);
    P2B_REQUIRE((align & 15) == 0, "all arrays must be 16-byte aligned");
    CfrParams p{};
    p.subgames = static_cast<const SubgameRec*>(subgames);
    p.nodes = static_cast<const NodeRecPacked*>(nodes);
    p.num_subgames = num_subgames;
    p.tables = tables;
    p.root_beliefs = root_beliefs;
    p.regrets = regrets;
    p.weight_sums = weight_sums;
    p.policy_avg = policy_avg;
    p.policy = policy;
    p.root_values = root_values;
    p.values_avg = values_avg;
    p.beliefs_avg = beliefs_avg;
    p.exploitability = exploitability;
    p.br_values = br_values;
    p.max_internal = max_internal;
    p.scalars = static_cast<const IterScalars*>(scalars);
    p.iterations = iterations;
    p.cfr_plus = flags & 1;
    p.enforce_zero_sum = (flags >> 1) & 1;
    p.cfr_avg = (flags >> 2) & 1;
    p.linear = (flags >> 4) & 1;
    p.init_depth = init_depth;
    p.rows = rows;
    return launch_cfr_solve_static(p, max_children, (cudaStream_t)stream);
}

}  // extern "C"
