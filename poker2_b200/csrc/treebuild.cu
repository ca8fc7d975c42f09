// Public betting trees built on the device: the breadth-first expansion that upstream runs
// level by level over the whole batch with dozens of small tensor ops per level
// (`SparseCFREvaluator._construct_subgame`, p2/search/sparse_cfr_evaluator.py:141-306, with the
// betting rules of `HUNLTensorEnv`: `legal_bins_amounts_and_mask` p2/env/hunl_tensor_env.py:348-423,
// `step` :766-992, `finish_and_assign_rewards` :707-724).
//
// Subgames are independent, so one warp expands one subgame: lane b evaluates bet bin b of the
// node at the head of the queue, a ballot orders the legal children, and the node records of the
// solver (cfr.cuh) come out directly in subgame-major breadth-first order together with each
// node's index in the upstream level-major order.  Two launches of the same code: a counting
// pass (sizes per subgame and per tree level), then, after prefix sums over the subgames, the
// pass that writes the records.
#include "cfr.cuh"
#include "common.cuh"

namespace p2b {

int sm_count();

namespace {

constexpr int kTreeWarps = 2;          // subgames per block (two node tables of kTreeMaxNodes states in static shared memory)
constexpr int kTreeMaxNodes = kCfrMaxNodes;  // what the solver kernel holds in shared memory
constexpr int kTreeMaxDepth = 63;
constexpr int kTreeMaxBetBins = 13;    // + fold, check/call, all-in <= 16 actions

// One subgame's root (16 x 32-bit words; the host packs it from its int64 arrays).
struct TreeRoot {
    int32_t to_act, pot, stack0, stack1, committed0, committed1, min_raise, actions_this_round;
    int32_t flags;  // 1: player 0 all-in, 2: player 1 all-in, 4: done
    int32_t street, button, start0, start1, raises, bb;
    float scale;
};
static_assert(sizeof(TreeRoot) == 64, "TreeRoot must be 64 bytes");

struct BetState {  // 32 bytes
    int32_t pot, stack[2], committed[2], min_raise;
    uint32_t small;  // to_act | flags << 8 | street << 16 | raises << 24
    int32_t actions_this_round;
};

struct TreeParams {
    const TreeRoot* roots;
    const int64_t* boards;  // [B][board_width], -1 = empty slot (records pass only)
    int board_width;
    int num_subgames;
    float bet_bins[kTreeMaxBetBins];
    int num_bet_bins;
    int max_depth;
    int max_raises;  // < 0: no cap
    // counting pass
    int32_t* counts;        // [B][8]: nodes, internal, model leaves, showdown leaves, max children, overflow, depth, 0
    int32_t* level_counts;  // [B][max_depth + 1]
    // records pass
    const int32_t* node_begin;  // [B]
    const int32_t* leaf_begin;  // [B]
    const int64_t* level_base;  // [B][max_depth + 1] level-major index of the subgame's first node of each level
    SubgameRec* subgames;
    NodeRecPacked* nodes;
    int64_t* to_level_major;  // [rows]
    int64_t* model_rows;      // [model leaves]
    int32_t* node_state;      // [rows][8] or null: pot, stack0, stack1, start0, start1, street, to_act, done
};

template <bool EMIT>
__global__ void __launch_bounds__(kTreeWarps * 32) tree_build_kernel(const TreeParams P) {
    __shared__ BetState s_state[kTreeWarps][kTreeMaxNodes];
    __shared__ uint32_t s_meta[kTreeWarps][kTreeMaxNodes];  // parent | action << 12 | depth << 20 (action 255: root)
    __shared__ float s_reward[kTreeWarps][kTreeMaxNodes];
    __shared__ int32_t s_level[kTreeWarps][kTreeMaxDepth + 1];
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int s = blockIdx.x * kTreeWarps + w;
    if (s >= P.num_subgames) return;
    BetState* st = s_state[w];
    uint32_t* meta = s_meta[w];
    float* reward = s_reward[w];
    int32_t* level = s_level[w];
    const TreeRoot root = P.roots[s];
    const int A = P.num_bet_bins + 3;
    for (int d = lane; d <= kTreeMaxDepth; d += 32) level[d] = 0;
    if (lane == 0) {
        BetState r;
        r.pot = root.pot;
        r.stack[0] = root.stack0; r.stack[1] = root.stack1;
        r.committed[0] = root.committed0; r.committed[1] = root.committed1;
        r.min_raise = root.min_raise;
        r.small = (uint32_t)root.to_act | ((uint32_t)root.flags << 8) | ((uint32_t)root.street << 16) | ((uint32_t)root.raises << 24);
        r.actions_this_round = root.actions_this_round;
        st[0] = r;
        meta[0] = 0u | (255u << 12);
        reward[0] = 0.0f;
    }
    __syncwarp();
    const long long row0 = EMIT ? P.node_begin[s] : 0;
    int n = 1, n_internal = 0, n_model = 0, n_showdown = 0, max_children = 0, overflow = 0, max_level = 0;
    for (int j = 0; j < n; ++j) {
        const BetState cur = st[j];
        const uint32_t m = meta[j];
        const int parent = m & 4095, action = (m >> 12) & 255, depth = (m >> 20) & 255;
        const int me = cur.small & 1, opp = 1 - me;
        const int flags = (cur.small >> 8) & 255, street = (cur.small >> 16) & 255, raises = cur.small >> 24;
        const bool done = flags & 4;
        const bool new_street = cur.actions_this_round == 0 && j != 0;
        const bool leaf = done || new_street || depth >= P.max_depth;
        // ---- legal bins (lane = bin) ----
        const int me_stack = cur.stack[me], opp_stack = cur.stack[opp];
        const int to_call = cur.committed[opp] - cur.committed[me];
        bool legal = false;
        int amount = -1;
        if (lane < A) {
            if (lane == 0) legal = to_call > 0;
            else if (lane == 1) legal = true;
            else if (lane == A - 1) {
                amount = me_stack;
                legal = me_stack > 0;
            } else {
                const int extra = (int)__fmul_rn(P.bet_bins[lane - 2], (float)cur.pot);  // fp32 product, truncated
                amount = to_call + extra;
                legal = me_stack > 0 && opp_stack > 0 && amount <= me_stack && extra >= cur.min_raise;
            }
            if (flags & (1 << opp)) legal = lane < 2;   // opponent all-in: fold or call only
            if (flags & (1 << me)) legal = lane == 1;   // actor all-in: call only
            if (P.max_raises >= 0 && lane >= 2) legal = legal && raises < P.max_raises;
        }
        const bool child = legal && !leaf;
        const unsigned cmask = __ballot_sync(0xffffffffu, child);
        const int k = __popc(cmask);
        if (n + k > kTreeMaxNodes) {
            overflow = 1;
            break;
        }
        // ---- children: the state after the action (lane = bin) ----
        if (child) {
            const int idx = n + __popc(cmask & ((1u << lane) - 1u));
            BetState nx = cur;
            int nflags = flags, nstreet = street, nraises = raises, nto_act = opp;
            float rew = 0.0f;
            int chips = 0;
            if (lane == 0) {
                nflags |= 4;
                const float share = opp == 0 ? (float)cur.pot : 0.0f;
                const float num = __fsub_rn(__fadd_rn((float)cur.stack[0], share), (float)root.start0);
                rew = __fdiv_rn(num, root.scale);
            } else if (lane == 1) {
                chips = min(to_call, me_stack);
            } else if (lane == A - 1) {
                chips = me_stack;
                nflags |= 1 << me;
            } else {
                chips = amount;
                nx.min_raise = max(cur.min_raise, chips - to_call);
            }
            nx.stack[me] -= chips;
            nx.committed[me] += chips;
            nx.pot += chips;
            if (lane >= 2) nraises += 1;
            nx.actions_this_round = cur.actions_this_round + 1;
            const int c0 = nx.committed[0], c1 = nx.committed[1];
            const bool a0 = nflags & 1, a1 = nflags & 2;
            const bool closed = !(nflags & 4) && (c0 == c1 || (a0 && a1) || (a0 && c0 <= c1) || (a1 && c1 <= c0)) &&
                                nx.actions_this_round >= 2;
            if (closed) {
                nx.committed[0] = nx.committed[1] = 0;
                nx.actions_this_round = 0;
                nto_act = 1 - root.button;
                nx.min_raise = root.bb;
                nraises = 0;
                if (street == 3) nflags |= 4;  // showdown
                nstreet = street + 1;
            }
            nx.small = (uint32_t)nto_act | ((uint32_t)nflags << 8) | ((uint32_t)nstreet << 16) | ((uint32_t)nraises << 24);
            st[idx] = nx;
            meta[idx] = (uint32_t)j | ((uint32_t)lane << 12) | ((uint32_t)(depth + 1) << 20);
            reward[idx] = rew;
        }
        // ---- this node's record ----
        const bool is_fold = action == 0 && done;
        const int kind = k > 0 ? 0 : (is_fold ? 1 : (street == 4 ? 2 : 3));
        const int rank_in_level = level[depth];
        if (EMIT && lane == 0) {
            NodeRecPacked rec;
            rec.parent = (uint16_t)parent;
            rec.first_child = (uint16_t)(k > 0 ? n : 0);
            rec.n_children = (uint8_t)k;
            rec.kind_act = (uint8_t)(kind | (me << 7));
            rec.depth = (uint8_t)depth;
            rec.internal_idx = (uint8_t)(kind == 3 ? n_model : n_internal);
            const float pot0 = (float)(cur.stack[0] + cur.pot - root.start0);
            rec.v0 = is_fold ? reward[j] : pot0;
            rec.v1 = (float)(cur.stack[1] + cur.pot - root.start1);
            P.nodes[row0 + j] = rec;
            P.to_level_major[row0 + j] = P.level_base[(long long)s * (P.max_depth + 1) + depth] + rank_in_level;
            if (kind == 3 && P.model_rows) P.model_rows[P.leaf_begin[s] + n_model] = row0 + j;
            if (P.node_state) {
                int32_t* o = P.node_state + (row0 + j) * 8;
                o[0] = cur.pot; o[1] = cur.stack[0]; o[2] = cur.stack[1]; o[3] = root.start0;
                o[4] = root.start1; o[5] = street; o[6] = me; o[7] = done ? 1 : 0;
            }
        }
        __syncwarp();
        if (lane == 0) level[depth] = rank_in_level + 1;
        __syncwarp();
        n_internal += kind == 0;
        n_model += kind == 3;
        n_showdown += kind == 2;
        max_children = max(max_children, k);
        max_level = max(max_level, depth);
        n += k;
    }
    if (!EMIT) {
        if (lane == 0) {
            int32_t* c = P.counts + (long long)s * 8;
            c[0] = n; c[1] = n_internal; c[2] = n_model; c[3] = n_showdown;
            c[4] = max_children; c[5] = overflow; c[6] = max_level; c[7] = 0;
        }
        for (int d = lane; d <= P.max_depth; d += 32) P.level_counts[(long long)s * (P.max_depth + 1) + d] = level[d];
    } else if (lane == 0) {
        SubgameRec sg;
        sg.node_begin = (int32_t)row0;
        sg.n_nodes = n;
        sg.n_internal = n_internal;
        sg.table_index = n_showdown > 0 ? s : -1;
        sg.scale = root.scale;
        unsigned long long mask = 0ull;
        int on_board = 0;
        for (int i = 0; i < P.board_width; ++i) {
            const long long c = P.boards[(long long)s * P.board_width + i];
            if (c >= 0 && c < 52) {
                mask |= 1ull << c;
                ++on_board;
            }
        }
        sg.board_mask = mask;
        const int n_allowed = (52 - on_board) * (51 - on_board) / 2;
        sg.allowed_prob = __fdiv_rn(1.0f, (float)max(n_allowed, 1));
        P.subgames[s] = sg;
    }
}

int fill_params(TreeParams& P, const void* roots, int num_subgames, const float* bet_bins, int num_bet_bins,
                int max_depth, int max_raises, const char* who) {
    if (!roots || (num_bet_bins > 0 && !bet_bins)) return set_error(P2B_ERR_ARG, "%s: null pointer", who);
    if (num_bet_bins < 0 || num_bet_bins > kTreeMaxBetBins)
        return set_error(P2B_ERR_ARG, "%s: %d bet bins; at most %d are supported", who, num_bet_bins, kTreeMaxBetBins);
    if (max_depth < 0 || max_depth > kTreeMaxDepth)
        return set_error(P2B_ERR_ARG, "%s: max_depth %d outside 0..%d", who, max_depth, kTreeMaxDepth);
    P = TreeParams{};
    P.roots = static_cast<const TreeRoot*>(roots);
    P.num_subgames = num_subgames;
    for (int i = 0; i < num_bet_bins; ++i) P.bet_bins[i] = bet_bins[i];
    P.num_bet_bins = num_bet_bins;
    P.max_depth = max_depth;
    P.max_raises = max_raises;
    return P2B_OK;
}

}  // namespace
}  // namespace p2b

using namespace p2b;

extern "C" {

int p2b_tree_count(const void* roots, int32_t num_subgames, const float* bet_bins, int32_t num_bet_bins,
                   int32_t max_depth, int32_t max_raises, int32_t* counts, int32_t* level_counts, void* stream) {
    if (num_subgames <= 0) return P2B_OK;
    TreeParams P;
    int rc = fill_params(P, roots, num_subgames, bet_bins, num_bet_bins, max_depth, max_raises, "p2b_tree_count");
    if (rc) return rc;
    if (!counts || !level_counts) return set_error(P2B_ERR_ARG, "p2b_tree_count: null pointer");
    P.counts = counts;
    P.level_counts = level_counts;
    const int grid = (num_subgames + kTreeWarps - 1) / kTreeWarps;
    tree_build_kernel<false><<<grid, kTreeWarps * 32, 0, (cudaStream_t)stream>>>(P);
    return check_cuda(cudaGetLastError(), "tree_build_kernel (count)");
}

int p2b_tree_records(const void* roots, const int64_t* boards, int32_t board_width, int32_t num_subgames,
                     const float* bet_bins, int32_t num_bet_bins, int32_t max_depth, int32_t max_raises,
                     const int32_t* node_begin, const int32_t* leaf_begin, const int64_t* level_base, void* subgames,
                     void* nodes, int64_t* to_level_major, int64_t* model_rows, int32_t* node_state, void* stream) {
    if (num_subgames <= 0) return P2B_OK;
    TreeParams P;
    int rc = fill_params(P, roots, num_subgames, bet_bins, num_bet_bins, max_depth, max_raises, "p2b_tree_records");
    if (rc) return rc;
    if (!boards || board_width < 0 || !node_begin || !leaf_begin || !level_base || !subgames || !nodes || !to_level_major)
        return set_error(P2B_ERR_ARG, "p2b_tree_records: null pointer");
    P.boards = boards;
    P.board_width = board_width;
    P.node_begin = node_begin;
    P.leaf_begin = leaf_begin;
    P.level_base = level_base;
    P.subgames = static_cast<SubgameRec*>(subgames);
    P.nodes = static_cast<NodeRecPacked*>(nodes);
    P.to_level_major = to_level_major;
    P.model_rows = model_rows;
    P.node_state = node_state;
    const int grid = (num_subgames + kTreeWarps - 1) / kTreeWarps;
    tree_build_kernel<true><<<grid, kTreeWarps * 32, 0, (cudaStream_t)stream>>>(P);
    return check_cuda(cudaGetLastError(), "tree_build_kernel (records)");
}

}  // extern "C"
