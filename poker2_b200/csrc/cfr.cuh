// Data structures of the fused subgame-CFR kernel (shared by cfr.cu and api.cu).
#pragma once

#include "common.cuh"

namespace p2b {

enum NodeKind : uint8_t { kInternal = 0, kFoldLeaf = 1, kShowdownLeaf = 2, kModelLeaf = 3 };

// One public-tree node as callers hand it in, 16 bytes.  Nodes of a subgame are stored breadth-first
// (parents before children, children of a node contiguous in action order); indices are local to
// the subgame.
struct NodeRecPacked {
    uint16_t parent;
    uint16_t first_child;
    uint8_t n_children;
    uint8_t kind_act;      // bits 0-1: NodeKind, bit 7: player to act
    uint8_t depth;
    uint8_t internal_idx;  // rank of this node among the internal nodes of its subgame (model leaf: rank
                           // among the model leaves of its subgame)
    float v0;              // fold leaf: value of player 0; showdown leaf: chips player 0 can win
    float v1;              // showdown leaf: chips player 1 can win
};
static_assert(sizeof(NodeRecPacked) == 16, "NodeRecPacked must be 16 bytes");

// The same node as the kernels keep it in shared memory.
struct NodeRec {
    uint16_t parent;
    uint16_t first_child;
    uint8_t n_children;
    uint8_t to_act;
    uint8_t kind;
    uint8_t depth;
    uint8_t internal_idx;
    float v0;
    float v1;
};
static_assert(sizeof(NodeRec) == 20, "NodeRec is five words");

__host__ __device__ __forceinline__ NodeRec unpack_node(const NodeRecPacked& r) {
    NodeRec n;
    n.parent = r.parent;
    n.first_child = r.first_child;
    n.n_children = r.n_children;
    n.to_act = r.kind_act >> 7;
    n.kind = r.kind_act & 3;
    n.depth = r.depth;
    n.internal_idx = r.internal_idx;
    n.v0 = r.v0;
    n.v1 = r.v1;
    return n;
}
__device__ __forceinline__ NodeRec load_node(const NodeRecPacked* p) {  // one 16-byte load
    const uint4 w = *reinterpret_cast<const uint4*>(p);
    NodeRecPacked r;
    *reinterpret_cast<uint4*>(&r) = w;
    return unpack_node(r);
}

struct SubgameRec {  // 32 bytes
    int32_t node_begin;   // first row of the subgame in the [rows][HPAD] state arrays
    int32_t n_nodes;
    int32_t n_internal;
    int32_t table_index;  // board-table blob of this subgame, -1 if it has no showdown leaf
    float scale;
    float allowed_prob;   // 1 / (number of combos not blocked by the board)
    unsigned long long board_mask;
};
static_assert(sizeof(SubgameRec) == 32, "SubgameRec must be 32 bytes");

// Per-iteration scalars, computed on the host in fp64 and rounded to fp32 the way the
// upstream Python code does (p2/search/cfr_evaluator.py:1346-1360, 285-303).
struct IterScalars {  // 32 bytes
    float num_pos, den_pos;  // t^alpha, t^alpha + 1      (regret discount, positive regrets)
    float num_neg, den_neg;  // t^beta,  t^beta + 1       (non-positive regrets)
    float mix_old, mix_new, mix_total;  // average-policy mixing weights and fl(old+new)
    int32_t do_mix;          // bit 0: 0 = average policy := current policy at this iteration; bits 1-2: linear CFR's
                             // alternating update, 1 + the player whose actions get no regret at this iteration
                             // (0: every action is updated); the lean iteration kernel never sees bits 1-2
};

constexpr int kCfrThreads = 672;  // 672 threads x 2 hands cover the 1344-float padded row
constexpr int kCfrMaxNodes = 320;   // nodes of one subgame (a depth-5 tree over {fold, call, two bets, all-in} has at most 273)
constexpr int kIterMaxNodes = 160;  // what the lean iteration kernel holds; larger subgames stay in the general kernel
constexpr int kCfrMaxChildren = 8;   // actions per node (fold, call, five bet sizes, all-in: the upstream dataclass default)
constexpr int kIterMaxChildren = 6;  // the lean iteration kernel's staging rows; batches with more stay in the general kernel

struct CfrParams {
    const SubgameRec* subgames;
    const NodeRecPacked* nodes;  // indexed by node_begin + local index
    int32_t num_subgames;
    const unsigned char* tables; // [*, kTabBytes] board tables
    const ComboTable* combos;    // filled in by the launcher
    const float* root_beliefs;   // [B][2][HPAD] input ranges (read-only)
    float* regrets;              // [rows][HPAD] cumulative regrets (out)
    float* weight_sums;          // [rows][HPAD] regret weight sums (out, may be null)
    float* policy_avg;           // [rows][HPAD] average policy (out)
    float* policy;               // [rows][HPAD] last current policy (out, may be null)
    float* root_values;          // [B][2][HPAD] values of the final average policy at the roots (out)
    float* values_avg;           // [rows][2][HPAD] the same for every node (out, may be null)
    float* beliefs_avg;          // [rows][2][HPAD] beliefs under the average policy (out, may be null)
    float* exploitability;       // [B] local exploitability of the average policy (out, may be null;
                                 // needs values_avg)
    float* br_values;            // [B][2] best-response value of each player at the root (out, may be null)
    float* scratch;              // per-block work rows
    long long scratch_stride;    // floats per block
    int32_t max_internal;        // largest n_internal over the batch
    const IterScalars* scalars;  // [iterations]
    int32_t iterations;
    int32_t cfr_plus;
    int32_t enforce_zero_sum;    // final pass: value outputs shifted to zero sum (cfr_evaluator.py:957-980, 1289-1292)
    int32_t cfr_avg;             // iteration passes: showdown values, regret weights and the beliefs handed to the
                                 // caller's model come from the beliefs under the average policy (:1029, :1133)
    int32_t linear;              // linear CFR (alternating updates, cfr_evaluator.py:1348-1349): the scalars carry the
                                 // skipped player per iteration; every pass stays in the general kernel
    int32_t iter_values;         // start and iteration passes store the values of every node in values_avg and (iteration
                                 // passes) the beliefs under the average policy in beliefs_avg: what a caller mixes into
                                 // running average values (`update_average_values`, cfr_evaluator.py:1260-1274)
    int32_t init_depth;          // depth of the deepest tree of the batch the subgames were built in
    int32_t* work_counter;       // dynamic subgame queue (zeroed by the launcher)
    const int32_t* queue_order;  // [B] subgame taken at each queue position (may be null: input order); a caller puts
                                 // the largest trees first so that the last blocks to finish hold small ones
    // ---- stepped mode: a launch runs part of the pass sequence and the state that a whole
    // solve keeps on chip is carried between launches in global memory.  Used when leaves are
    // valued by a caller-side model between the two sweeps of a pass.  All zero / null in
    // the one-launch mode.
    int32_t stepped;             // 0: one launch runs every pass
    int32_t pass_begin;          // first pass of this launch (-1 = start pass, iterations = final pass)
    int32_t pass_end;            // last pass of this launch (inclusive)
    int32_t phases;              // bit 0: top-down sweep, bit 1: bottom-up sweep (+ best responses after
                                 // the final pass); 4 alone: only the best responses, from the state the final
                                 // pass left and the leaf values in values_avg; 8 alone: the best-response pass of a
                                 // `model_br` warm start, after the start pass (values_avg holds its node values)
    float* carry_sums;           // [rows][2] normalisation sums of the node beliefs ([2][rows][2] with cfr_avg or iter_values)
    float* carry_roots;          // [B][4][HPAD] prior (2 rows) and root beliefs (2 rows) of the pass
    const int32_t* leaf_begin;   // [B] first model-leaf slot of each subgame
    float* leaf_beliefs;         // [slots][2][HPAD] beliefs at the model leaves (out, top-down sweep)
    const float* leaf_values;    // [slots][2][HPAD] values at the model leaves (in, bottom-up sweep)
    // ---- inputs of leaf sampling (p2/search/cfr_evaluator.py:1336-1341, sparse_cfr_evaluator.py:325-426)
    const int32_t* sample_pass;  // [B] pass whose current policy is kept in policy_sample (may be null)
    float* policy_sample;        // [rows][HPAD] (out, may be null)
    float* beliefs_last;         // [rows][2][HPAD] beliefs of the last iteration at internal nodes (out, may be null)
    const float* start_policy;   // [rows][HPAD] policy of the start pass (may be null: uniform over the children)
    float warm_weight;           // one-call solve only: > 0 = warm start of type `model` (cfr_evaluator.py:913-926) after the
                                 // start pass, weight = warm-start iterations x multiplier; scalars[0] then belongs to the
                                 // warm start's own policy update
    // ---- limits the record check compares the records with
    long long rows;              // rows of the state arrays
    int32_t leaf_slots;          // model-leaf slots of leaf_beliefs / leaf_values
    // ---- a one-launch solve split over several launches (start pass, iteration passes, final pass)
    int32_t scratch_per_block;   // stepped launch whose work rows are not carried: one set per block
    int32_t large_only;          // general kernel: skip the subgames the lean iteration kernel holds (it skips the others)
};

// floats of scratch one block needs: per internal node reach[2], average reach[2], values[2]
__host__ __device__ inline long long cfr_scratch_floats(int max_internal) {
    return (long long)max_internal * 6 * P2B_HPAD;
}

// `fast_scratch`: the scratch area also holds the hand-over rows of a split solve
// (cfr_solve_scratch_floats), so a plain solve may run its iteration passes in cfr_iter_kernel.
int launch_cfr_solve(const CfrParams& p, int num_blocks, int max_children, cudaStream_t stream, bool fast_scratch = false);
long long cfr_iter_scratch_floats(int max_internal, int max_children);
long long cfr_solve_scratch_floats(int max_internal, int max_children, int num_blocks, int num_subgames, long long rows);
int launch_cfr_iter(const CfrParams& p, int num_blocks, cudaStream_t stream);
int cfr_path_policy(int policy);  // returns the previous one; < 0 only queries
int cfr_iteration_timing(int enable);
int cfr_iteration_ms(float* ms);
int cfr_default_blocks();
int launch_cfr_solve_static(const CfrParams& p, int max_children, cudaStream_t stream);
int launch_cfr_warm_seed(const NodeRecPacked* nodes, long long rows, const float* start_policy, float weight, float* regrets,
                         float* weight_sums, cudaStream_t stream);
long long cfr_static_scratch_floats();
int cfr_static_status(int32_t* host_status, cudaStream_t stream);

}  // namespace p2b
