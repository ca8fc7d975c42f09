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

/* showdown_ev_triton (src/p2/search/fused_cfr_triton.py:2271-2320): the EV of every strength-sorted
 * position straight from sorted-order inputs, `rows` rows of `hands` (<= 1344) entries each:
 * b_sorted fp32 opponent range in strength order, c1_sorted / c2_sorted int32 hole cards of the
 * position (0..51; anything else counts as no card), l_idx / r_idx int32 tie group [L,R) of the
 * position.  out [rows,hands] fp32 = win/den - loss/den with the formula of _showdown_value
 * (cfr_evaluator.py:544-596), 0 where den <= eps.  The caller permutes back, masks the hands on
 * the board and scales by the pot, as upstream. */
int p2b_showdown_ev_sorted(const float* b_sorted, const int32_t* c1_sorted, const int32_t* c2_sorted,
                           const int32_t* l_idx, const int32_t* r_idx, int64_t rows, int32_t hands,
                           float eps, float* out, void* stream);

/* ---- fused subgame CFR (src/p2/search/cfr_evaluator.py:1497-1528 evaluate_cfr with
 * cfr_iteration :1331-1381, on the ragged tree of sparse_cfr_evaluator.py:141-306) ----
 * One persistent kernel runs the start pass, `iterations` DCFR iterations and the final
 * average-policy evaluation for `num_subgames` independent subgames whose leaves are all
 * terminal (fold or showdown).  Rows are 1344 floats (1326 combos + 18 padding floats) so
 * that every row is 16-byte aligned; all row arrays must be 16-byte aligned.
 *
 *  subgames   [num_subgames] 32-byte records {int32 node_begin, n_nodes, n_internal,
 *             table_index; float scale, allowed_prob; uint64 board_mask}
 *  nodes      [rows] 16-byte records {uint16 parent, first_child; uint8 n_children, kind_act
 *             (bits 0-1 kind: 0 internal, 1 fold leaf, 2 showdown leaf, 3 other leaf; bit 7 the
 *             player to act; the other bits zero), depth, internal_idx; float v0, v1},
 *             breadth-first per subgame, local indices.  A subgame has at most 320 nodes (a
 *             depth-5 tree over {fold, call, two bet sizes, all-in} has at most 273); subgames of
 *             up to 160 nodes run their iteration passes in the lean kernel, larger ones in the
 *             general kernel, within the same call; max_children <= 8, and a batch with more than
 *             6 children at some node runs every pass in the general kernel
 *  tables     showdown tables from p2b_rank_hands, indexed by table_index
 *  root_beliefs [num_subgames,2,1344] input ranges
 *  regrets, weight_sums (may be NULL), policy_avg, policy (may be NULL): [rows,1344] out
 *  root_values [num_subgames,2,1344] out; values_avg, beliefs_avg [rows,2,1344] out (may be NULL)
 *  exploitability [num_subgames], br_values [num_subgames,2] out (may be NULL; need values_avg):
 *             local exploitability of the average policy and the best-response value of each
 *             player at the root (cfr_evaluator.py:718-764)
 *  rows       number of rows of the state arrays (the record check refuses subgames that reach past it)
 *  scratch    at least p2b_cfr_scratch_floats(max_internal, num_blocks) floats of work space.  With
 *             p2b_cfr_solve_scratch_floats(max_internal, max_children, num_blocks, num_subgames, rows)
 *             floats the solve runs as
 *             three launches (start pass; iteration passes in a leaner kernel; final pass) with the same
 *             results, bit for bit; the extra floats carry the root rows between the launches (very
 *             small batches stay in the one-launch form, see p2b_cfr_path_policy)
 *  scalars    [iterations] 32-byte records {float t^alpha, t^alpha+1, t^beta, t^beta+1,
 *             mix_old, mix_new, fl(mix_old+mix_new); int32 do_mix (bit 0; bits 1-2 see flags bit 4)}
 *  flags      bit 0: CFR+ (cumulative regrets clamped at zero after every update, cfr_evaluator.py:1366-1368);
 *             bit 1: the value outputs of the final pass (root_values, values_avg) are shifted to zero
 *             sum, per node minus the mean over the players of sum_h values * beliefs_avg, except at
 *             terminal nodes -- what upstream does when model.enforce_zero_sum is set
 *             (_maybe_enforce_zero_sum :957-980 at the end of update_average_values_final :1289-1292);
 *             the best responses then start from the shifted leaf values, as upstream;
 *             bit 2: `cfr_avg` upstream (cfr_evaluator.py:1029, :1133): in the iteration passes the showdown
 *             values, the regret weights and the leaf_beliefs handed to the caller's model are taken at the
 *             beliefs under the average policy instead of the current one (the de-averaging of the model's
 *             values, :997-1018, is the caller's part of set_leaf_values); such a solve keeps every pass in
 *             the general kernel;
 *             bit 4: linear CFR (alternating updates, cfr_evaluator.py:1348-1349): the `do_mix` word of every
 *             scalars record then carries, in bits 1-2, 1 + the player whose actions get no regret at that
 *             iteration; such a solve keeps every pass in the general kernel;
 *             bit 3 (p2b_cfr_step only): the bottom-up sweep of the start pass and of every iteration pass stores
 *             the values of every node in values_avg and (iteration passes) the beliefs under the average
 *             policy, at inner nodes and at the leaves a model values, in beliefs_avg -- the inputs of the
 *             running value average upstream keeps when value_targets_from_final_policy is off (:1260-1274)
 *  init_depth depth of the deepest tree of the batch (the upstream start pass re-normalises
 *             every belief row once per level of the batch-wide tree)
 *  work_counter four int32, zeroed by the call: [0] the queue the thread blocks take subgames
 *             from; [1] status; [2], [3] internal.  Before every launch a checking kernel compares
 *             every subgame's records with the solver's limits (1..320 nodes per subgame, all
 *             inside the `rows` rows, 1..8 children per internal node, children stored after their
 *             parent and inside the subgame, internal_idx < max_internal, unused record bits zero, root
 *             internal, a table for every showdown leaf, a slot for every model leaf).
 *             On a violation status = 1 + the index of an offending subgame and NOTHING is
 *             solved (outputs untouched); otherwise status stays 0
 *  num_blocks 0 = one block per SM
 *  sample_pass [num_subgames] int32 (may be NULL), policy_sample [rows,1344] out (may be NULL):
 *             the current policy of pass sample_pass[s] is kept for subgame s -- the
 *             policy_probs_sample snapshot of cfr_evaluator.py:1336-1341 (taken at the start of
 *             iteration t_sample, i.e. the policy of pass t_sample-1); rows of subgames whose
 *             sample_pass is outside 0..iterations-1 are left untouched
 *  beliefs_last [rows,2,1344] out (may be NULL): beliefs of the last iteration at the internal
 *             nodes (what sample_leaves returns for the sampled nodes).
 *  queue_order [num_subgames] int32 (may be NULL: input order): the subgame taken at each position of the
 *             queue the thread blocks draw from.  A permutation with the largest trees first shortens the
 *             tail in which few blocks are still busy; results do not depend on it.
 *  start_policy [rows,1344] (may be NULL: uniform over the children): the policy of the start pass, i.e. the
 *             soft-max of the model's policy head at every node (initialize_policy_and_beliefs :832-886)
 *  warm_start_weight  0, or warm-start iterations x multiplier: after the start pass the regrets are seeded so
 *             that regret matching replays the start policy (warm_start of type `model`, :913-926).  scalars[0]
 *             then belongs to the warm start's own policy update (update_policy(w), :923) and scalars[k], k >= 1,
 *             to iteration w + k - 1; `iterations` counts these passes.  Needs the scratch area of
 *             p2b_cfr_solve_scratch_floats. */
int p2b_cfr_solve(const void* subgames, const void* nodes, int32_t num_subgames, int64_t rows, int32_t max_children,
                  int32_t max_internal, const unsigned char* tables, const float* root_beliefs,
                  float* regrets, float* weight_sums, float* policy_avg, float* policy,
                  float* root_values, float* values_avg, float* beliefs_avg, float* exploitability,
                  float* br_values, float* scratch, int64_t scratch_floats, const void* scalars, int32_t iterations, int32_t flags,
                  int32_t init_depth, int32_t* work_counter, int32_t num_blocks, const int32_t* sample_pass,
                  float* policy_sample, float* beliefs_last, const int32_t* queue_order, const float* start_policy,
                  float warm_start_weight, void* stream);
int64_t p2b_cfr_scratch_floats(int32_t max_internal, int32_t num_blocks);
int64_t p2b_cfr_solve_scratch_floats(int32_t max_internal, int32_t max_children, int32_t num_blocks,
                                     int32_t num_subgames, int64_t rows);
int p2b_cfr_default_blocks(void);
/* Which kernel runs the iteration passes of a p2b_cfr_solve whose leaves are all terminal (process-wide
 * setting, no counterpart in the upstream project).  0, the default: the lean kernel, except for batches so
 * small that the general kernel is quicker (at most one subgame per SM; or fewer than eight per SM while
 * max_internal x max_children + 1 exceeds 160, i.e. some subgame may be too large for the lean kernel).
 * 1: the lean kernel whenever it applies.  Results are the same bits either way.  Returns the previous
 * setting; a negative argument only queries. */
int p2b_cfr_path_policy(int32_t policy);
/* Measurement aid (no counterpart in the upstream project): with timing enabled on the current
 * device, a p2b_cfr_solve that runs its iteration passes in the lean kernel brackets that one
 * launch with CUDA events on the caller's stream; p2b_cfr_iteration_ms waits for it and writes
 * its duration in milliseconds to the HOST float *ms. */
int p2b_cfr_iteration_timing(int32_t enable);
int p2b_cfr_iteration_ms(float* ms);

/* p2b_cfr_step -- part of a solve, for subgames whose non-terminal leaves (start of the next
 * street, depth limit) are valued by the caller's model (set_leaf_values,
 * src/p2/search/cfr_evaluator.py:1025-1047): the model runs between the top-down sweep of a
 * pass (policy, reach, beliefs) and its bottom-up sweep (values, regrets).  Passes are
 * numbered -1 (start pass), 0..iterations-1 (DCFR iterations), iterations (final evaluation
 * of the average policy).  A call runs the passes pass_begin..pass_end; `phases` selects the
 * top-down sweep (1), the bottom-up sweep (2) or both (3); with 1 or 2 the range is one pass; 4 (with
 * pass_begin = pass_end = iterations) runs only the best responses, from the state the final pass left and
 * the leaf values found in values_avg; 8 (with pass_begin = pass_end = -1, after a start pass run with flags
 * bit 3) is the best-response pass of a warm start of type `model_br` (cfr_evaluator.py:927-955): it sets the
 * regrets of every child to unblocked(other player's start beliefs) x (best-response value of the child for the
 * player who acted - that player's value of the parent under the start policy); the caller multiplies by
 * warm_start_iterations x multiplier, sets the weight sums to that factor and goes on with pass 0.
 * 16 (with pass_end = pass_begin + 1) joins the bottom-up sweep of pass_begin and the top-down sweep of the
 * next pass in one launch: nothing happens on the host between them unless the caller wants it to, and a
 * block then visits a subgame once per pass instead of twice (same results; no faster in our measurements,
 * the time of a pass is the walk over the subgames).
 * The caller's loop is: for every pass { step(pass, 1); leaf_values = model(leaf_beliefs);
 * step(pass, 2); }, or step(-1, 1); for every pass { leaf_values = model(leaf_beliefs);
 * pass == iterations ? step(pass, 2) : step(pass..pass+1, 16); }.  Arrays as in p2b_cfr_solve, plus state
 * carried between calls:
 *  scratch      p2b_cfr_scratch_floats(max_internal, 1) * num_subgames floats (one set of
 *               work rows per subgame instead of per block)
 *  carry_sums   [rows,2] floats ([2,rows,2] with flags bit 2 or 3), carry_roots [num_subgames,4,1344] floats (opaque)
 *  leaf_begin   [num_subgames] int32: first leaf slot of each subgame; a node of kind 3 uses
 *               slot leaf_begin[subgame] + its internal_idx field; leaf_slots = number of slots
 *  leaf_beliefs [slots,2,1344] out (top-down sweep): both players' beliefs at each such leaf
 *  leaf_values  [slots,2,1344] in (bottom-up sweep): both players' values there, in the units
 *               of the other leaf values (chips / scale)
 * With leaf_beliefs == NULL / leaf_values == NULL such leaves are skipped / valued 0.
 * queue_order (may be NULL) as in p2b_cfr_solve: the order in which the blocks take the subgames; the
 * largest trees first shortens a launch over a ragged batch (192 subgames of 9..237 nodes: 35.8 against
 * 41.8 ms for 24 iterations). */
int p2b_cfr_step(const void* subgames, const void* nodes, int32_t num_subgames, int64_t rows, int32_t max_children,
                 int32_t max_internal, const unsigned char* tables, const float* root_beliefs,
                 float* regrets, float* weight_sums, float* policy_avg, float* policy,
                 float* root_values, float* values_avg, float* beliefs_avg, float* exploitability,
                 float* br_values, float* scratch, int64_t scratch_floats, const void* scalars,
                 int32_t iterations, int32_t flags, int32_t init_depth, int32_t* work_counter,
                 int32_t num_blocks, int32_t pass_begin, int32_t pass_end, int32_t phases,
                 float* carry_sums, float* carry_roots, const int32_t* leaf_begin, int32_t leaf_slots,
                 float* leaf_beliefs, const float* leaf_values, const int32_t* sample_pass, float* policy_sample,
                 float* beliefs_last, const int32_t* queue_order, const float* start_policy, void* stream);

/* Start policy and warm start (initialize_policy_and_beliefs with a policy head,
 * src/p2/search/cfr_evaluator.py:830-886, and warm_start of type `model`, :887-926).
 * start_policy [rows,1344] (last argument of p2b_cfr_step, may be NULL = uniform): the policy of
 * the start pass, one row per non-root node.  p2b_cfr_warm_seed is called between the start
 * pass (pass -1, both sweeps) and pass 0 of a stepped solve: per non-root row it sets
 * regrets = start_policy * w and weight_sums = w (may be NULL) with w = weight * mean over the
 * 1326 hands of max(regret, 0), the regrets being those the start pass left in `regrets`;
 * weight = warm_start_iterations * warm_start_multiplier.  The caller's scalars array then
 * starts at the warm-start iteration (see solver.SteppedSolver). */
int p2b_cfr_warm_seed(const void* nodes, int64_t rows, const float* start_policy, float weight, float* regrets,
                      float* weight_sums, void* stream);

/* Public betting trees built on the device (replaces the level-by-level tensor expansion of
 * `SparseCFREvaluator._construct_subgame`, src/p2/search/sparse_cfr_evaluator.py:141-306, with
 * the betting rules of src/p2/env/hunl_tensor_env.py:348-423 (legal bins), :766-992 (step) and
 * :707-724 (fold reward)); one warp expands one subgame breadth-first.
 *
 * roots [num_subgames][16] 32-bit words per subgame: to_act, pot, stack0, stack1, committed0,
 * committed1, min_raise, actions_this_round, flags (1: player 0 all-in, 2: player 1 all-in,
 * 4: done), street (0..3), button, starting_stack0, starting_stack1, raises made on the street,
 * big blind, scale (fp32 bits).  bet_bins: HOST array of num_bet_bins (<= 13) pot fractions;
 * actions are {fold, check/call, fractions..., all-in}.  max_depth <= 63.  max_raises < 0: no cap
 * (the cap is not an upstream option).
 *
 * p2b_tree_count: counts [num_subgames][8] = nodes, internal nodes, leaves valued by a model,
 * showdown leaves, largest child count, overflow flag (more nodes than the solver kernel supports,
 * 320), depth of the tree, 0; level_counts [num_subgames][max_depth+1] nodes per tree level.
 * p2b_tree_records: given the exclusive prefix sums over the subgames of the node counts
 * (node_begin), of the model-leaf counts (leaf_begin) and, per level, of the level counts offset by
 * the level's start in the upstream level-major order (level_base [num_subgames][max_depth+1]),
 * writes the 32-byte subgame records, the 16-byte node records (subgame-major, breadth-first),
 * to_level_major [rows] (upstream index of every row), model_rows [model leaves] (row of every
 * model leaf, slot order; may be NULL when there is none) and, when node_state is not NULL, [rows][8] int32 = pot, stack0, stack1,
 * starting_stack0, starting_stack1, street, to_act, done.  boards [num_subgames][board_width] int64
 * card ids, -1 = empty slot. */
int p2b_tree_count(const void* roots, int32_t num_subgames, const float* bet_bins, int32_t num_bet_bins,
                   int32_t max_depth, int32_t max_raises, int32_t* counts, int32_t* level_counts, void* stream);
int p2b_tree_records(const void* roots, const int64_t* boards, int32_t board_width, int32_t num_subgames,
                     const float* bet_bins, int32_t num_bet_bins, int32_t max_depth, int32_t max_raises,
                     const int32_t* node_begin, const int32_t* leaf_begin, const int64_t* level_base, void* subgames,
                     void* nodes, int64_t* to_level_major, int64_t* model_rows, int32_t* node_state, void* stream);

/* p2b_cfr_solve_noalloc -- the same solve without any allocation.  (No counterpart in the
 * upstream project: it exists for hosts of this library that cannot allocate.)
 *
 * Who needs it: a data-generation worker that was handed a fixed slice of GPU memory by
 * its trainer and must not take more; a caller in a latency-sensitive loop, for which a
 * cudaMalloc would stall the whole device; a process whose framework allocator already
 * owns all free memory, so that a driver allocation could simply fail.  Such a caller
 * cannot provide the work rows and the queue counter that p2b_cfr_solve asks for, and
 * must not trigger the one-time table allocation that the other entry points perform.
 *
 * This variant keeps its work rows, queue counter and combo table in a fixed area that is
 * part of the library image: 32 MiB (p2b_cfr_noalloc_scratch_floats() floats) on every
 * GPU that loads the library, held until the process exits.  Limits that follow:
 *   - a subgame needs max_internal * 6 * 1344 floats of work rows per thread block; if
 *     that exceeds the area the call fails with a message and nothing is launched;
 *   - the number of thread blocks is what fits in the area (at most one per SM), so large
 *     trees run on fewer SMs than with p2b_cfr_solve.
 * The first call on a device resolves the area's addresses and uploads a 2.6 KB table
 * with a blocking copy (under a lock, so first calls from several threads are safe); make
 * that first call before any stream capture.  Every call uses
 * the same area: it zeroes the queue counter itself and needs no other clearing, but two
 * calls that overlap on the GPU (different streams or threads) race on it -- serialise them.
 * It calls no cudaMalloc / cudaFree and no allocating library routine; inputs and outputs
 * are the caller's, with the meaning they have in p2b_cfr_solve.
 *
 * The record check's verdict lives in the same area.  p2b_cfr_noalloc_status waits for
 * `stream`, then copies it to the HOST word *status: 0, or 1 + the index of a subgame whose
 * records were refused, in which case the last call solved nothing.  It allocates nothing. */
int p2b_cfr_solve_noalloc(const void* subgames, const void* nodes, int32_t num_subgames, int64_t rows,
                          int32_t max_children, int32_t max_internal, const unsigned char* tables,
                          const float* root_beliefs, float* regrets, float* weight_sums,
                          float* policy_avg, float* policy, float* root_values, float* values_avg,
                          float* beliefs_avg, float* exploitability, float* br_values, const void* scalars,
                          int32_t iterations, int32_t flags, int32_t init_depth, void* stream);
int64_t p2b_cfr_noalloc_scratch_floats(void);
int p2b_cfr_noalloc_status(int32_t* status, void* stream);

/* ---- step-level kernels (src/p2/search/fused_cfr_triton.py) ----------------------------
 * One entry point per fused kernel of the upstream module, on caller-owned contiguous fp32
 * tensors in the upstream node order; index tensors are int64, masks one byte per entry.
 * Iteration-dependent scalars are read from device memory.  H is the row length (1326). */
/* fused_dcfr_update_with_tensors_ (:200-235); scalars4 = {t^a, t^b, t^a+1, t^b+1} */
int p2b_step_dcfr_update(const float* regrets, float* cumulative, float* weight_sums, float* positive_out,
                         const float* scalars4, int64_t n, int apply_dcfr, int cfr_plus, void* stream);
/* fused_block_and_normalize_beliefs_ (:286-335) */
int p2b_step_block_normalize(float* target, const uint8_t* allowed, const float* allowed_prob, int64_t rows,
                             int32_t rows_per_outer, int32_t H, float eps, void* stream);
/* fused_regret_matching_divide_ (:369-399) */
int p2b_step_regret_matching_divide(const float* positive, const float* denom, const float* uniform, float* out,
                                    int64_t n, float eps, void* stream);
/* fused_weight_child_values (:438-477) */
int p2b_step_weight_child_values(const float* values, const int64_t* prev_actor, const float* policy_hero,
                                 const float* policy_opp, float* out, int64_t M, int32_t H, void* stream);
/* fused_update_average_values_with_tensors_ (:538-560) */
int p2b_step_update_average_values(float* values_avg, const float* latest, const float* old_w, const float* new_w,
                                   const float* inv_total, int64_t n, void* stream);
/* fused_avg_values_zero_sum_ (:623-668) with subtract_b=0, scale=1/(old+new);
 * fused_model_values_mix_zero_sum (:1739-1775) with subtract_b=1, scale=NULL:
 * out = (a*coef_a +/- b*coef_b) [*scale] - 0.5*sum_p sum_h out*beliefs (rows of [2,H]).
 * subtract_b: bit 0 = subtract b's term, bit 1 = divide by *scale instead of multiplying (the non-fused
 * `update_average_values`, cfr_evaluator.py:1260-1274, divides by old + new).
 * enforce_zero_sum: 0 = no shift; 1 = the sum accumulated in fp64; 2 (H = 1326, or rows padded to 1344) = two fp32 sums in the
 * order of the CPU row reduction the non-fused upstream code goes through (cfr_evaluator.py:973-976) */
int p2b_step_mix_zero_sum(const float* a, const float* b, const float* beliefs, const uint8_t* ignore,
                          const float* coef_a, const float* coef_b, const float* scale, float* out, int64_t rows,
                          int32_t H, int subtract_b, int enforce_zero_sum, void* stream);
/* fused_model_values_mix_with_tensors (:1658-1680): out = coef_a*a - coef_b*b */
int p2b_step_scaled_difference(const float* a, const float* b, const float* coef_a, const float* coef_b, float* out,
                               int64_t n, void* stream);
/* fused_regret_tail_ (:712-766) */
int p2b_step_regret_tail(const float* values_achieved, const float* actor_values, const float* src_weights,
                         const int64_t* parent_index, const int64_t* prev_actor, float* regrets, int64_t bottom,
                         int64_t total, int32_t H, void* stream);
/* fused_average_policy_mix_with_tensors_ (:879-914) */
int p2b_step_average_policy_mix(const float* reach, const float* reach_avg, const float* policy, float* policy_avg,
                                const int64_t* to_act, const int64_t* parent_index, const float* old_w,
                                const float* new_w, const float* total_w, int64_t bottom, int64_t total, int32_t H,
                                float eps, void* stream);
/* fused_parent_sum (:1279-1313) and fused_sibling_sum (:1355-1398, broadcast_to_children=1) */
int p2b_step_parent_sum(const float* values, const int64_t* child_offsets, const int64_t* child_count, float* out,
                        int64_t num_parents, int32_t H, int broadcast_to_children, int64_t out_offset, void* stream);
/* fused_divide_by_parent_sum_ (:1316-1352) */
int p2b_step_divide_by_parent_sum(const float* pos, const float* fallback, const float* parent_sum,
                                  const int64_t* parent_index, float* out, int64_t num_children, int32_t H, float eps,
                                  void* stream);
/* unblocked_mass_triton (:1110-1157) and unblocked_mass_opp_at_parents_triton (:1067-1107):
 * out[r] = unblocked mass of the 1326-float row src + row_index[r]*1326 (row_index NULL = r) */
int p2b_step_unblocked_mass(const float* src, const int64_t* row_index, float* out, int64_t rows, void* stream);
/* unblocked_mass_ratio_triton (:1559-1602) and unblocked_mass_ratio_indirect_triton (:1499-1556) */
int p2b_step_unblocked_mass_ratio(const float* numer, const float* denom, const int64_t* parent_index, float* out,
                                  int64_t rows, float eps, void* stream);
/* fused_weighted_parent_sum (:1838-1889) */
int p2b_step_weighted_parent_sum(float* values, const int64_t* prev_actor, const float* policy_hero,
                                 const float* policy_opp, const int64_t* child_offsets, const int64_t* child_count,
                                 int64_t parent_base, int64_t num_parents, int32_t H, void* stream);
/* fused_reach_weights_depth_ (:1944-1986) */
int p2b_step_reach_weights(float* reach, const float* policy, const uint8_t* allowed, const int64_t* parent_index,
                           const int64_t* prev_actor, int64_t start, int64_t end, int32_t H, void* stream);
/* fused_deep_beliefs_ (:2039-2092) */
int p2b_step_deep_beliefs(float* out, const float* root_beliefs, const float* reach, const float* allowed_prob,
                          const int64_t* root_index, int64_t num_roots, int64_t total, int32_t H, float eps,
                          void* stream);

/* ---- chance nodes (src/p2/search/chance_node_helper.py:359-479, single_card_chance_values) --
 * p2b_chance_expand: for each root b, one sample per card not on its board (ascending card
 * id; samples grouped by root).  boards [num_roots, board_len] int64 with -1 for empty
 * slots; sample_offsets [num_roots+1] int64 = exclusive prefix of the number of free cards;
 * pre_beliefs [num_roots,2,1326].  Outputs per sample: post_beliefs [S,2,1326] (combos
 * touching the extended board zeroed, rows renormalised, uniform fallback at mass <= 1e-12,
 * :434-444), root_lookup [S] int64 and board_samples [S, board_len] int64 (:402-418). */
int p2b_chance_expand(const float* pre_beliefs, const int64_t* boards, int32_t board_len, const int64_t* sample_offsets,
                      int64_t num_roots, int64_t num_samples, float* post_beliefs, int64_t* root_lookup,
                      int64_t* board_samples, void* stream);
/* Fused forms for a bf16 value network (same arithmetic as the two calls around them, no
 * fp32 copy of the expanded beliefs).  p2b_chance_expand_features writes the network's input
 * rows: features [num_samples, feature_stride] bf16 = both players' post-card beliefs (2 x 1326),
 * the 52-d one-hot of the extended board, the root's 3 context scalars (context [num_roots,3]
 * fp32), zeros up to feature_stride (>= 2707).  The two belief rows of a root are player_stride
 * floats apart (1326 packed, 1344 for the solver's padded rows).  root_lookup may be NULL.
 * p2b_indexed_mean_bf16: out[r, p, h] = mean over the samples sample_offsets[r]..[r+1] of
 * src[sample, p*1326 + h] (bf16 rows src_stride apart), fp32, ascending sample order; the two
 * output rows of a root are out_player_stride floats apart. */
int p2b_chance_expand_features(const float* pre_beliefs, int64_t player_stride, const int64_t* boards,
                               int32_t board_len, const int64_t* sample_offsets, int64_t num_roots,
                               int64_t num_samples, const float* context, void* features_bf16,
                               int64_t feature_stride, int64_t* root_lookup, void* stream);
int p2b_indexed_mean_bf16(const void* src_bf16, int64_t src_stride, const int64_t* sample_offsets,
                          int64_t num_roots, float* out, int64_t out_player_stride, void* stream);
/* Flop chance node (src/p2/search/chance_node_helper.py:218-357).  p2b_expand_on_boards:
 * post_beliefs [num_roots*num_boards, 2, 1326] = the beliefs of every root re-blocked and
 * re-normalised on every given board (boards [num_boards, board_len] int64, -1 = empty slot;
 * sample = root*num_boards + board; uniform fallback at mass <= 1e-12, :262-284).
 * p2b_mean_over_hand_perms: out[n, h] = mean over p of values[n, perms[p, h]] (perms
 * [num_perms, 1326] int32: the hole-card index permutation of each suit permutation), added in
 * ascending p -- `_avg_over_perms` (:17-27); rows are packed 1326-float rows. */
int p2b_expand_on_boards(const float* pre_beliefs, int64_t player_stride, const int64_t* boards, int32_t board_len,
                         int64_t num_roots, int64_t num_boards, float* post_beliefs, void* stream);
int p2b_mean_over_hand_perms(const float* values, const int32_t* perms, int32_t num_perms, int64_t rows,
                             float* out, void* stream);
/* p2b_indexed_add_rows: out[index[i], :] (+)= src[i, :] in ascending i, for a sorted int64
 * index (the index_add_ of :468-475); mean != 0 divides by max(count,1) (:476-477);
 * accumulate == 0 overwrites out instead of adding to it. */
int p2b_indexed_add_rows(float* out, const int64_t* index, const float* src, int64_t num_src, int64_t num_out,
                         int64_t width, int mean, int accumulate, void* stream);

/* ---- self-test (no counterpart in the reference) ------------------------------------------
 * The solver's divisions share divisors and run through a short correctly rounded sequence
 * (csrc/exactdiv.cuh).  p2b_selftest_division compares it with the compiler's IEEE division
 * on at least num_pairs generated (x, y) pairs of stream `seed` and ADDS the number of
 * results that differ in any bit to *mismatches and the number of pairs served by the short
 * sequence to *short_path (device pointers, cleared by the caller). */
int p2b_selftest_division(uint64_t num_pairs, uint32_t seed, unsigned long long* mismatches,
                          unsigned long long* short_path, void* stream);
/* Directed form: all 2^23 divisor mantissas at five exponents (both ends of the valid range
 * included), each against 16 numerators placed on rounding boundaries (1, the largest mantissa, the
 * divisor one ulp up and down, its mirrored mantissa, a neighbouring exponent, pseudo-random ones).
 * ADDS the differing results to *mismatches and the quotients compared to *checked. */
int p2b_selftest_division_sweep(unsigned long long* mismatches, unsigned long long* checked, void* stream);

#ifdef __cplusplus
}
#endif
#endif
