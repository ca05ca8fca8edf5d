/*
 * thrml_b200.h — C ABI of libthrml_b200: a block-Gibbs sampling engine for NVIDIA B200 (sm_100a).
 *
 * The library replaces, for thrml-rs's sampling path, everything from
 * BlockSamplingProgram::sample_single_block downward (crates/thrml-samplers/src/program.rs:324-393),
 * i.e. the Burn/WGPU tensor dispatch, the per-block samplers and the observers' per-sample work.
 * The Rust-level types (Node, Block, BlockSpec, InteractionGroup, BlockGibbsSpec, ...) stay the
 * caller's; they are flattened to the integer arrays this header takes.
 *
 * Conventions
 *  - every function returns an int32 status: THRML_OK or a negative THRML_ERR_*; nothing throws or
 *    aborts.  thrml_last_error() returns a thread-local message for the last failing call; the
 *    messages keep the substrings thrml-rs's own tests look for ("same type", "twice",
 *    "leading dimension", "tail node blocks", "n_spin", "empty", "Number of samplers", ...).
 *  - the caller owns every host buffer it passes; the library copies during the call and owns all
 *    device memory until the matching *_destroy.
 *  - a handle is used by one host thread at a time; distinct handles are independent.
 *  - no function falls back to the CPU: without a usable CUDA device every device function returns
 *    THRML_ERR_CUDA.  The thrml_rng_*, thrml_builder_*, thrml_lattice_* and thrml_greedy_coloring
 *    functions are host-only and work without a GPU.
 *
 * Node ids are dense per builder: 0 .. n_nodes-1.  A node kind is 0 for NodeType::Spin and K >= 1 for
 * NodeType::Categorical{n_categories: K} (crates/thrml-core/src/node.rs:8-21).
 *
 * State values follow the reference: a spin is 0 or 1 (1 means +1), a categorical node holds its
 * category index (crates/thrml-samplers/src/spin_gibbs.rs:618-637, softmax.rs:60-97).  On the device a
 * node's state is one byte per chain, chains innermost: state[class][global position][chain].
 */
#ifndef THRML_B200_H
#define THRML_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define THRML_OK 0
#define THRML_ERR_INVALID_ARG (-1)
#define THRML_ERR_BAD_COLOURING (-2)
#define THRML_ERR_CUDA (-3)
#define THRML_ERR_NCCL (-4)
#define THRML_ERR_TIMEOUT (-5)
#define THRML_ERR_OOM (-6)
#define THRML_ERR_UNSUPPORTED (-7)

/* sampler kinds, one per free block (crates/thrml-samplers/src/sampler.rs:58-71 is the trait they implement) */
#define THRML_SAMPLER_SPIN_GIBBS 0        /* SpinGibbsConditional, spin_gibbs.rs:59-100 */
#define THRML_SAMPLER_CATEGORICAL_GIBBS 1 /* CategoricalGibbsConditional, softmax.rs:228-271 */
#define THRML_SAMPLER_SOFTMAX 2           /* SoftmaxConditional, softmax.rs:103-222: logits = the block's per-category weights summed \
                                             over active slots (tables whose weights are not [rows, K, 1] are skipped, neighbour  \
                                             states are not read), then the same Gumbel-argmax draw */

typedef struct thrml_ctx thrml_ctx;
typedef struct thrml_builder thrml_builder;
typedef struct thrml_program thrml_program;
typedef struct thrml_state thrml_state;
typedef struct thrml_moments thrml_moments;
typedef struct thrml_comm thrml_comm;

/* Message of the last failing call on this thread (empty string if none). */
const char* thrml_last_error(void);
/* Library version string. */
const char* thrml_version(void);

/* ------------------------------------------------------------------------------------------------
 * RngKey — crates/thrml-samplers/src/rng.rs:10-51
 * split(n): n == 0 -> nothing written; n == 1 -> out[0] = key (rng.rs:24-26); else a ChaCha8 stream
 * seeded with rand_core 0.6's seed_from_u64(key) gives n successive next_u64() values (rng.rs:29-36).
 * ---------------------------------------------------------------------------------------------- */
int32_t thrml_rng_split(uint64_t key, int64_t n, uint64_t* out);

/* ------------------------------------------------------------------------------------------------
 * Input generators used by the benchmark configurations (host only).
 * thrml_lattice_edges: nearest-neighbour square lattice of make_nearest_neighbor_lattice
 *   (crates/thrml-models/src/graph_utils.rs:177-243): side rounded up to even, nodes row-major, one edge
 *   (min,max) per neighbour pair; the reference's HashSet order is replaced by ascending (min,max).
 *   edges_out holds 2*n_edges ids; pass NULL to query the count only.  colour_out[i] = (row+col)%2.
 * thrml_greedy_coloring: greedy_coloring of crates/thrml-examples/src/lib.rs:114-147 — nodes visited in
 *   index order, smallest colour not used by an already coloured neighbour.
 * ---------------------------------------------------------------------------------------------- */
int32_t thrml_lattice_edges(int64_t side_len, int32_t torus, int64_t* side_out, int64_t* n_edges_out,
                            int64_t* edges_out, int32_t* colour_out);
int32_t thrml_greedy_coloring(int64_t n_nodes, int64_t n_edges, const int64_t* edges, int32_t* colour_out,
                              int32_t* n_colours_out);

/* ------------------------------------------------------------------------------------------------
 * Program builder = the host-side index compiler.
 *   BlockGibbsSpec::new           crates/thrml-samplers/src/program.rs:28-64
 *   BlockSpec::new                crates/thrml-core/src/blockspec.rs:15-66
 *   InteractionGroup::new         crates/thrml-core/src/interaction.rs:128-181
 *   to_interaction_groups         crates/thrml-models/src/discrete_ebm.rs:379-510
 *   BlockSamplingProgram::new     crates/thrml-samplers/src/program.rs:88-318
 * ---------------------------------------------------------------------------------------------- */
/* kinds[n_nodes]; dtype_order lists node kinds in the insertion order of the caller's
 * node_shape_dtypes map: it fixes the numbering of the global-state classes (blockspec.rs:19-28). */
int32_t thrml_builder_create(const int32_t* kinds, int64_t n_nodes, const int32_t* dtype_order,
                             int32_t n_dtype_order, thrml_builder** out);
void thrml_builder_destroy(thrml_builder* b);
/* Free blocks are appended in order; blocks that share `superblock` are updated from the same
 * pre-update state (sampling.rs:40-59).  superblock ids must be non-decreasing. */
int32_t thrml_builder_add_free_block(thrml_builder* b, const int64_t* nodes, int64_t n, int32_t superblock,
                                     int32_t sampler_kind);
int32_t thrml_builder_add_clamped_block(thrml_builder* b, const int64_t* nodes, int64_t n);
/* One InteractionGroup: head[rows]; tails[n_tails][rows] (the first n_spin tails are spin blocks, the
 * rest categorical); w[rows][d1][d2] f32. */
int32_t thrml_builder_add_interaction_group(thrml_builder* b, const int64_t* head, int64_t rows,
                                            const int64_t* tails, int32_t n_tails, int32_t n_spin,
                                            const float* w, int32_t d1, int32_t d2);
/* One DiscreteEBMFactor (SpinEBMFactor / CategoricalEBMFactor are the special cases):
 * spin_groups[n_spin_groups][rows], cat_groups[n_cat_groups][rows], w[rows][d1][d2]; appends the directed
 * interaction groups the reference derives (discrete_ebm.rs:379-510). n_groups_out may be NULL. */
int32_t thrml_builder_add_discrete_factor(thrml_builder* b, const int64_t* spin_groups, int32_t n_spin_groups,
                                          const int64_t* cat_groups, int32_t n_cat_groups, int64_t rows,
                                          const float* w, int32_t d1, int32_t d2, int32_t* n_groups_out);
/* IsingEBM::get_factors (crates/thrml-models/src/ising.rs:105-143): bias factor over `nodes` with beta*b,
 * edge factor with beta*J; either may be empty. */
int32_t thrml_builder_add_ising(thrml_builder* b, const int64_t* nodes, int64_t n_nodes, const float* biases,
                                const int64_t* edges, int64_t n_edges, const float* weights, float beta);
/* Runs BlockSpec::new + BlockSamplingProgram::new. */
int32_t thrml_builder_compile(thrml_builder* b);

/* Introspection of the compiled tables (the bit-exact parity surface). */
int32_t thrml_builder_counts(const thrml_builder* b, int32_t* n_free, int32_t* n_clamped, int32_t* n_groups_total,
                             int32_t* n_classes);
int32_t thrml_builder_node_location(const thrml_builder* b, int64_t node, int32_t* sd_index, int64_t* position);
/* Interaction group g of the builder's flat list: sizes, then contents (any out pointer may be NULL). */
int32_t thrml_builder_group_shape(const thrml_builder* b, int32_t g, int64_t* rows, int32_t* n_tails,
                                  int32_t* n_spin, int32_t* d1, int32_t* d2);
int32_t thrml_builder_group_data(const thrml_builder* b, int32_t g, int64_t* head, int64_t* tails, float* w);
/* Number of compiled (non-empty) tables of free block `block`, then table t of that block:
 * k = padded slot count, wdim = d1*d2, n = block length. */
int32_t thrml_builder_block_tables(const thrml_builder* b, int32_t block, int32_t* n_tables, int64_t* n_nodes);
int32_t thrml_builder_table_shape(const thrml_builder* b, int32_t block, int32_t t, int32_t* k, int32_t* wdim,
                                  int32_t* n_spin, int32_t* n_tails, int32_t* source_group);
/* rows[n*k] (interaction_slices), active[n*k], w[n*k*wdim], idx[n_tails][n*k] (global positions),
 * tail_sd[n_tails] (class of each tail) — program.rs:159-300. */
int32_t thrml_builder_table_data(const thrml_builder* b, int32_t block, int32_t t, int32_t* rows, uint8_t* active,
                                 float* w, int32_t* idx, int32_t* tail_sd);

/* ------------------------------------------------------------------------------------------------
 * Device context, program, state.
 * ---------------------------------------------------------------------------------------------- */
/* One context = one CUDA device + one stream (one process per GPU is the intended deployment). */
int32_t thrml_ctx_create(int32_t device_id, thrml_ctx** out);
void thrml_ctx_destroy(thrml_ctx* ctx);
int32_t thrml_ctx_synchronize(thrml_ctx* ctx);

/* The two steps before the sampling path, on the device.
 * thrml_builder_compile_device: same result as thrml_builder_compile, table for table and byte for byte; the layout
 *   (BlockSpec::new, crates/thrml-core/src/blockspec.rs:15-66) stays on the host, the slot tables of
 *   BlockSamplingProgram::new (crates/thrml-samplers/src/program.rs:88-318) are built per interaction group by a stable
 *   radix sort of (head node, row), a run-length scan for the slot numbers and one scatter, then read back into the builder.
 * thrml_greedy_coloring_device: same colours as thrml_greedy_coloring (crates/thrml-examples/src/lib.rs:114-147), computed
 *   as a dataflow over the edges directed from lower to higher node index; n_passes_out (may be NULL) receives the number
 *   of passes launched, a multiple of 8 that bounds the longest index-increasing path of the graph from above. */
int32_t thrml_builder_compile_device(thrml_builder* b, thrml_ctx* ctx);
int32_t thrml_greedy_coloring_device(thrml_ctx* ctx, int64_t n_nodes, int64_t n_edges, const int64_t* edges,
                                     int32_t* colour_out, int32_t* n_colours_out, int32_t* n_passes_out);
/* Failure-detection self test (no reference counterpart; the reference's errors are Result<_, String> / panics): a
 * kernel waits on a pipeline barrier that nothing signals; its bounded wait runs out, it returns, and this call
 * reports THRML_ERR_TIMEOUT.  The context remains usable. */
int32_t thrml_debug_wait_timeout(thrml_ctx* ctx);
/* cudaStream_t of the context, for callers that time with their own events. */
void* thrml_ctx_stream(thrml_ctx* ctx);

/* ------------------------------------------------------------------------------------------------
 * Multi-GPU (no counterpart in the reference, which drives one device from one thread): one process per GPU, one
 * thrml_comm per process = one rank of a NCCL communicator.  NCCL is loaded at run time (libnccl.so.2) by the first of
 * these calls; a failing NCCL call returns THRML_ERR_NCCL with NCCL's message.  Rank 0 calls thrml_comm_unique_id and the
 * host distributes the 128 bytes to the other ranks by its own means (a file, a socket, MPI, torch.distributed ...);
 * every rank then calls thrml_comm_create (collective: returns once all world_size ranks have joined).
 * thrml_comm_adopt wraps an ncclComm_t the host already owns (it is not destroyed with the handle).
 * ---------------------------------------------------------------------------------------------- */
#define THRML_COMM_ID_BYTES 128
int32_t thrml_comm_unique_id(uint8_t* id_out /* [THRML_COMM_ID_BYTES] */);
int32_t thrml_comm_create(thrml_ctx* ctx, const uint8_t* id, int32_t rank, int32_t world_size, thrml_comm** out);
int32_t thrml_comm_adopt(thrml_ctx* ctx, void* nccl_comm, thrml_comm** out);
void thrml_comm_destroy(thrml_comm* c);
int32_t thrml_comm_info(const thrml_comm* c, int32_t* rank_out, int32_t* world_out, int32_t* nccl_version_out);

/* Uploads the compiled tables.  The program snapshots the weights (as the reference does,
 * program.rs:216-235); thrml_program_update_weights refreshes table t of a block explicitly. */
int32_t thrml_program_create(thrml_ctx* ctx, const thrml_builder* b, thrml_program** out);
void thrml_program_destroy(thrml_program* p);
int32_t thrml_program_update_weights(thrml_program* p, int32_t block, int32_t t, const float* w);
/* The same refresh without the host-side gather: every table compiled from interaction group `group` (its index in the
 * builder's flat list — groups are appended in the order of the add_* calls, thrml_builder_counts reports how many exist)
 * re-reads its slot weights on the device from the group's parameter rows: slot s takes
 * scale * w[(row(s) mod period)][0 .. wdim), row(s) as in program.rs:216-235.  w: host, [period][wdim], in the group's own
 * weight layout.  The group of a factor with S spin node groups repeats the factor's rows S times (discrete_ebm.rs:391-453),
 * hence `period`: for a model built by thrml_builder_add_ising, the bias factor's group takes b[N] with period N and the
 * edge factor's group takes J[E] with period E, both with scale = beta — an SGD step (train_mnist.rs:616-732,
 * IsingEBM::update_weights, ising.rs:71-86) uploads N + E floats.  Derived tables are rebuilt on the device. */
int32_t thrml_program_update_group(thrml_program* p, int32_t group, const float* w, int64_t period, int32_t wdim, float scale);
/* Per-program tuning options (no counterpart in the reference; results never depend on them, tests use them to run
 * every route).  They belong to the handle: other programs and other host threads are not affected.
 *   THRML_OPT_DENSE_TILES   tile shape of the dense (tensor-core) kernels: 1 = CTA pairs sharing 256-row tiles through
 *                           tcgen05 cta_group::2 (each CTA stages half of the B operand), 0 = one CTA per 128-row tile,
 *                           2 (the default) = chosen per launch from the shape (pairs for long reductions without much
 *                           row padding).
 *   THRML_OPT_SPLIT_MARGIN  widens (units of 2^-24 of probability, >= 0) the window around each draw's probability inside
 *                           which the split-field-table update of sequential-sum nodes recomputes the field in the
 *                           canonical order; 0 (the default) keeps the derived bound, 2^25 sends every draw through the
 *                           exact route.  Setting it rebuilds the affected blocks' tables.
 *   THRML_OPT_GATHER_ONLY   1 = blocks whose default kernel is the general spin kernel (kind 7) or the register-resident
 *                           categorical kernels (kinds 5 and 8) run the node x four-chain gather kernels (kinds 0 and 2) instead;
 *                           0 (the default) = each block's own kernel.  The states are the same either way.
 *   THRML_OPT_STATE_FORMAT  0 (the default) = sweeps read and write the state as one byte per spin and chain; 1 = when every
 *                           free block runs the threshold-table kernel (kind 1), nothing is staged and the state holds at
 *                           least 1009 chains, sweeps (and a moment observer whose rows the update kernels own) run on a
 *                           bit-packed mirror of the spin state (1.125 bytes of traffic per update instead of 9, the same
 *                           noise, the same states); the byte copy is brought up to date by the first call that needs
 *                           it (downloads, other observers, energies, uploads), and the mirror by the next sweep. */
#define THRML_OPT_DENSE_TILES 1
#define THRML_OPT_SPLIT_MARGIN 2
#define THRML_OPT_GATHER_ONLY 3
#define THRML_OPT_STATE_FORMAT 4
int32_t thrml_program_set_option(thrml_program* p, int32_t option, double value);
int32_t thrml_program_get_option(const thrml_program* p, int32_t option, double* value_out);
/* Dense bipartite path.  A spin block whose neighbours all lie in one other spin block (a layer of an RBM-style model:
 * IsingEBM with bipartite edges, crates/thrml-models/src/ising.rs:105-143, which the reference samples as a padded
 * gather, program.rs:159-300) can compute its local fields as one tensor-core GEMM against the other block's +-1 states
 * instead.  Couplings are held as bf16 with f32 accumulation; allow_bf16_rounding = 0 refuses blocks whose couplings are
 * not already bf16 values.  The sum order differs from the gather kernel's, so a draw can differ where the uniform falls
 * within rounding distance of the threshold.  n_blocks_out = number of blocks switched (kernel kind 3). */
int32_t thrml_program_enable_dense(thrml_program* p, int32_t allow_bf16_rounding, int32_t* n_blocks_out);
/* Which kernel a free block runs: 0 generic gather kernel, 1 threshold-table kernel (spin blocks whose
 * nodes have at most 8 single-spin-tail slots), 2 categorical kernel, 3 dense tensor-core kernel, 4 sequential-sum
 * kernel (spin blocks with single-spin-tail slots, more than 8 active slots on some node), 5 categorical kernel for nodes with
 * at most 8 active slots (slot data held in registers, Gumbel noise screened with fast logarithms), 6 a spin block that
 * mixes kinds 1 and 4 node by node (at least a quarter of its nodes have at most 8 neighbour slots), 7 the general spin
 * kernel (slots whose tail is a product of up to three spins or a categorical node that selects the weight, at most 32
 * active slots per node; warp per node, 16 chains per lane), 8 categorical kernel for nodes with 9 to 32 active slots and
 * at most 16 categories (slot data in shared memory, logits in registers). */
int32_t thrml_program_block_kernel(const thrml_program* p, int32_t block, int32_t* kind_out);

/* n_chains chains held on this device; chain_offset = global id of local chain 0 (the in-kernel random
 * stream is a function of the global chain id, so results do not depend on how chains are sharded). */
int32_t thrml_state_create(thrml_program* p, int64_t n_chains, int64_t chain_offset, thrml_state** out);
void thrml_state_destroy(thrml_state* s);
/* Block index runs over free blocks then clamped blocks.  Host layout [chain][node], f32 as in the
 * reference (0/1 or category index) or raw bytes. */
int32_t thrml_state_upload_f32(thrml_state* s, int32_t block, const float* host);
int32_t thrml_state_download_f32(thrml_state* s, int32_t block, float* host);
int32_t thrml_state_upload_u8(thrml_state* s, int32_t block, const uint8_t* host);
int32_t thrml_state_download_u8(thrml_state* s, int32_t block, uint8_t* host);
/* Chains [chain_begin, chain_begin + n_chains) of one block only: host[chain - chain_begin][node]. */
int32_t thrml_state_download_chains_u8(thrml_state* s, int32_t block, int64_t chain_begin, int64_t n_chains, uint8_t* host);
/* Several blocks per call (block ids in `blocks`, one host pointer each): all copies and layout kernels are queued on the
 * context's stream and the host waits once at the end.  _u8_many: hosts[i] = [chain][node] bytes as in
 * thrml_state_upload_u8.  _packed (spin blocks only; the mirror of thrml_sample_states_packed): bits[i] = [node][word] u32,
 * word w = chains 32w .. 32w+31, bit c & 31 — one bit per spin over the host link, no transpose on the device.
 * No counterpart in the reference, whose states are f32 tensors (crates/thrml-core/src/state_tree.rs:32-73). */
int32_t thrml_state_upload_u8_many(thrml_state* s, const int32_t* blocks, int32_t n_blocks, const uint8_t* const* hosts);
int32_t thrml_state_upload_packed(thrml_state* s, const int32_t* blocks, int32_t n_blocks, const uint32_t* const* bits);
/* Device-to-device copy of one block's state between two states of the same program and chain count (asynchronous on
 * the context's stream; the reference's equivalent is cloning a state tensor, e.g. sampling.rs:237). */
int32_t thrml_state_copy_block(thrml_state* dst, const thrml_state* src, int32_t block);
/* Same result as thrml_state_upload_u8, for hosts that must not allocate device memory while running (their GPU memory
 * is already committed to another runtime's pool, or a cudaMalloc's device-wide synchronisation would stall them).
 * No counterpart in the reference.  The [chain][node] bytes are staged in a fixed 4 MiB array inside the library image
 * (held on every GPU that loads the library until exit) instead of a growable buffer: nodes x chains of the block must
 * not exceed 4 MiB (4194304), larger blocks are rejected with THRML_ERR_INVALID_ARG.  The call allocates nothing.  The
 * first call on a device looks up the array's device address; make it before any stream capture begins.  All calls
 * share the array (it keeps the previous call's bytes, none of which are read): calls whose GPU work could overlap on
 * one device race and must be issued one after the other. */
int32_t thrml_state_upload_u8_static(thrml_state* s, int32_t block, const uint8_t* host);

/* hinton_init (crates/thrml-models/src/ising.rs:602-673): for each listed block, P(s=1) = sigmoid(beta*b)
 * (not 2*beta*b, ising.rs:650), s = (u <= p).  biases = concatenation of the listed blocks' biases.
 * inj_u (nullable, host): uniforms [block][chain][node] to use instead of the in-kernel stream. */
int32_t thrml_hinton_init(thrml_state* s, const int32_t* blocks, int32_t n_blocks, const float* biases, float beta,
                          uint64_t key, const float* inj_u);
/* Uniform random state for every free block (spins: fair bits; categorical: uniform category). */
int32_t thrml_state_randomize(thrml_state* s, uint64_t key);

/* Injected noise (host pointer, f32), consumed in update order: for every sweep, for every free block in
 * sampling order, a spin block takes u[node][chain] and a categorical block takes u[node][category][chain].
 * Both sides of a parity test feed the same stream. */
typedef struct thrml_noise {
    const float* u;
    int64_t len;
} thrml_noise;

/* sample_blocks (sampling.rs:28-63): one sweep; per-block keys = key.split(n_free_blocks). */
int32_t thrml_sample_blocks(thrml_state* s, uint64_t key, const thrml_noise* inj);
/* run_blocks (sampling.rs:81-106): n_iters sweeps with keys = key.split(n_iters). */
int32_t thrml_run_blocks(thrml_state* s, uint64_t key, int64_t n_iters, const thrml_noise* inj);
/* IsingEBM::energy / energy_batched (crates/thrml-models/src/ising.rs:150-321): per chain
 * E = -beta (sum_i b_i s_i + sum_(i,j) J_ij s_i s_j) with s = 2x - 1, accumulated in f64.  nodes[n_nodes] with biases,
 * edges[2*n_edges] (node id pairs) with weights; energy_out[n_chains] on the host. */
int32_t thrml_ising_energy(thrml_state* s, int64_t n_nodes, const int64_t* nodes, const float* biases, int64_t n_edges,
                           const int64_t* edges, const float* weights, float beta, double* energy_out);
/* DiscreteEBMFactor::factor_energy (crates/thrml-models/src/discrete_ebm.rs:552-592) for every chain of the state:
 * E = -sum over rows of W[row][c_1][c_2] * prod over the spin groups of (2x - 1), accumulated in f64 in a fixed order.
 * nodes[(n_spin_groups + n_cat_groups) * rows]: node ids, one run of `rows` per group, spin groups first; w[rows*d1*d2];
 * categorical group k indexes axis k (no categorical group: d1 = d2 = 1; one: d2 = 1; at most two, the weights being
 * rank 3).  A category at or beyond the axis length reads the last entry.  energy_out[n_chains] on the host.
 * The energy of a FactorizedEBM (ebm.rs:109-130) is the sum of this over its factors. */
int32_t thrml_factor_energy(thrml_state* s, int64_t rows, int32_t n_spin_groups, int32_t n_cat_groups, const int64_t* nodes, const float* w, int32_t d1, int32_t d2,
                            double* energy_out);
/* sample_single_block (program.rs:324-393): update one free block in place; `key` is the block's own key. */
int32_t thrml_sample_single_block(thrml_state* s, int32_t block, uint64_t key);
/* <s_a s_b> over this device's chains for every node pair of two spin blocks (s = 2x-1): host_out[n_a][n_b] f32, computed
 * exactly from integer counts on the tensor cores.  The pairwise form of the second moments of
 * MomentAccumulatorObserver::ising_moment_spec (moment.rs:125-148) for a complete bipartite edge set. */
int32_t thrml_pair_correlation(thrml_state* s, int32_t block_a, int32_t block_b, float* host_out);
/* One CD-1 step on a two-layer model (the data/model phases of estimate_kl_grad, ising.rs:531-594, collapsed to one
 * sweep): upload v0 (host [chain][visible node] 0/1, nullable = keep the current visible state), h0 ~ P(h|v0) with
 * key.split(2)[0], pos = <v0 h0>, one sweep sample_blocks(key.split(2)[1]), neg = <v1 h1>.  pos/neg: host
 * [n_visible][n_hidden] f32, nullable. */
int32_t thrml_cd1_step(thrml_state* s, int32_t visible_block, int32_t hidden_block, const uint8_t* v0_host, uint64_t key,
                       float* pos_host, float* neg_host);
/* Bring-up check of the CTA-pair tensor-core kernels (no reference counterpart): after a pair launch on this state, both
 * CTAs of a pair must have been given the same tensor-memory base address; THRML_ERR_CUDA if they differ. */
int32_t thrml_debug_pair_tmem_check(thrml_state* s);
/* thrml_cd1_step with the visible data held in another state of the same program and chain count (a resident data set that
 * many steps start from): `data`'s visible block is read for h0 and <v0 h0> and is not modified; v1 and h1 land in `s`. */
int32_t thrml_cd1_step_from(thrml_state* s, thrml_state* data, int32_t visible_block, int32_t hidden_block, uint64_t key, float* pos_host,
                            float* neg_host);
/* thrml_cd1_step_from with the chains sharded over the ranks of `comm` (the chain-parallel form of the step: every rank
 * holds its own data and chain states, whose chain offsets give the global chain ids): the correlation matrices returned on
 * every rank are the means over all ranks' chains (one ncclAllReduce of 2 x n_visible x n_hidden f32 and a scale; exact when
 * the chain count per rank is a power of two).  The hidden block must be on the dense path. */
int32_t thrml_cd1_step_comm(thrml_state* s, thrml_state* data, int32_t visible_block, int32_t hidden_block, uint64_t key, thrml_comm* comm,
                            float* pos_host, float* neg_host);
/* Local field gamma[chain][node] (spin block) or logits theta[chain][node][K] (categorical block) of a free
 * block in the current state — spin_gibbs.rs:512-611 / softmax.rs:586-709. */
int32_t thrml_fields_debug(thrml_state* s, int32_t block, float* out);

/* ------------------------------------------------------------------------------------------------
 * Observers.
 * MomentAccumulatorObserver (crates/thrml-observers/src/moment.rs:52-148,157-237): running sums of
 * prod f(x) over listed node tuples, f = 2x-1 when transform_to_spin.  spec = n_types moment types,
 * rows_per_type[t] rows each, row r holds members[row_ptr[r] .. row_ptr[r+1]) (node ids).  Sums run over
 * samples and over this device's chains, exactly (int64).
 * ---------------------------------------------------------------------------------------------- */
int32_t thrml_moments_create(thrml_program* p, int32_t n_types, const int64_t* rows_per_type, const int64_t* row_ptr,
                             const int64_t* members, int32_t transform_to_spin, thrml_moments** out);
void thrml_moments_destroy(thrml_moments* m);
int32_t thrml_moments_reset(thrml_moments* m);
/* observe(): add the current state's products (moment.rs:205-233). */
int32_t thrml_moments_observe(thrml_moments* m, thrml_state* s);
/* sums_out[rows_per_type[type]] as int64 totals; n_obs_out = observations * local chains. */
int32_t thrml_moments_read(thrml_moments* m, int32_t type, int64_t* sums_out, int64_t* n_obs_out);
/* Device pointer of the int64 accumulators of all types, concatenated, and their count — the buffer a
 * multi-GPU host hands to its single allreduce(sum). */
int32_t thrml_moments_device_buffer(thrml_moments* m, void** dev_ptr_out, int64_t* count_out);
int32_t thrml_moments_add_observations(thrml_moments* m, int64_t n_obs);
/* The single collective of the chain-parallel deployment (chains sharded over the ranks of `comm`, program replicated,
 * noise keyed by the global chain id): adds the sums and the observation count over all ranks, in place on every rank,
 * with ncclAllReduce on the context's stream.  Collective: every rank calls it with an observer of the same spec.  The
 * sums travel as int32 when the reduced observation counts prove that every total fits, else as int64.  The reduction of
 * the sums is asynchronous; thrml_moments_read waits for it. */
int32_t thrml_moments_allreduce(thrml_moments* m, thrml_comm* comm);
/* How the rows are served when the observer follows a sweep: rows the update kernels accumulate themselves (single
 * spins and neighbour pairs of threshold-table blocks) and rows left to the separate observer kernel. */
int32_t thrml_moments_fused_info(const thrml_moments* m, int64_t* n_fused_rows, int64_t* n_other_rows);
/* Kernel launches this state has issued for block updates so far: ordinary per-block launches, and launches of the
 * persistent multi-sweep kernel that small all-threshold-table programs use inside thrml_run_blocks /
 * thrml_sample_with_observation / thrml_sample_states_packed (one launch covers up to 4096 block updates).
 * No counterpart in the reference; hosts use it to count launches and tests to see which path ran. */
int32_t thrml_state_launch_counts(const thrml_state* s, int64_t* block_launches, int64_t* persistent_launches);

/* Per-node category counts for the nodes of the listed blocks (counts[node][category], int64), the
 * category-marginal observable of the Potts configuration.  K = table width. */
int32_t thrml_marginals_create(thrml_program* p, const int32_t* blocks, int32_t n_blocks, int32_t K,
                               thrml_moments** out);

/* sample_with_observation (sampling.rs:178-320): key.split_two -> warm-up, observe, then n_samples-1 times
 * (steps_per_sample sweeps, observe).  moments may be NULL.  obs_blocks/obs_out (nullable) = StateObserver
 * (state_observer.rs:25-47): obs_out[sample][observed node][chain] bytes, observed nodes = concatenation of
 * the listed blocks.  Total sweeps = n_warmup + (n_samples-1)*steps_per_sample. */
int32_t thrml_sample_with_observation(thrml_state* s, uint64_t key, int64_t n_warmup, int64_t n_samples,
                                      int64_t steps_per_sample, thrml_moments* moments, const int32_t* obs_blocks,
                                      int32_t n_obs_blocks, uint8_t* obs_out, const thrml_noise* inj);

/* estimate_kl_grad (crates/thrml-models/src/ising.rs:531-594): key.split_two -> (key_pos, key_neg); each phase is
 * estimate_moments (ising.rs:455-505) = sample_with_observation with a MomentAccumulatorObserver over
 * ising_moment_spec(bias_nodes, weight_edges); the gradient -beta (mean_pos - mean_neg) is formed on the device and only
 * the two gradient vectors come back.  `pos` / `neg`: states of the positive and the negative program (IsingTrainingSpec,
 * ising.rs:392-433) already holding their initial free-block states and their clamped blocks (for `pos` the data row the
 * reference picks, row key_pos mod batch of each data array, ising.rs:549-559, then the conditioning values; for `neg` the
 * conditioning values).  moments_pos / moments_neg: observers created on the respective programs with the same two moment
 * types (single nodes, then pairs); they are reset first.  Means divide by samples x chains.  grad_w_out[n_edges],
 * grad_b_out[n_nodes]: host f32, either may be NULL. */
int32_t thrml_estimate_kl_grad(thrml_state* pos, thrml_state* neg, thrml_moments* moments_pos, thrml_moments* moments_neg, uint64_t key,
                               int64_t warmup_pos, int64_t samples_pos, int64_t steps_pos, int64_t warmup_neg, int64_t samples_neg, int64_t steps_neg,
                               float beta, float* grad_w_out, float* grad_b_out);

/* sample_states (sampling.rs:128-156) with the StateObserver output (state_observer.rs:25-47) streamed bit-packed:
 * bits_out[sample][observed node][word] (host, u32), word w = chains 32w .. 32w+31, bit c & 31; observed nodes = the
 * listed spin blocks concatenated; max(n_samples, 1) samples are written. */
int32_t thrml_sample_states_packed(thrml_state* s, uint64_t key, int64_t n_warmup, int64_t n_samples, int64_t steps_per_sample,
                                   const int32_t* obs_blocks, int32_t n_obs_blocks, uint32_t* bits_out);

/* ------------------------------------------------------------------------------------------------
 * Implicit lattice: a height x width periodic nearest-neighbour Ising lattice with one coupling and one bias, sampled
 * with the two checkerboard blocks, state bit-packed (32 spins per word, chains innermost), held as a stripe of rows
 * [row_begin, row_begin + n_rows) plus one halo row above and below.  It samples exactly what IsingSamplingProgram
 * (crates/thrml-models/src/ising.rs:342-388) would on make_nearest_neighbor_lattice's torus
 * (crates/thrml-models/src/graph_utils.rs:177-243) with blocks [(row+col) even, (row+col) odd] — same fields, same
 * noise, same states — for lattices whose per-node tables (program.rs:101-134) could never be built.
 * One sweep (sampling.rs:28-63): keys = key.split(2); update colour 0 with keys[0], refresh colour 0's halo rows in the
 * neighbouring stripes, update colour 1 with keys[1], refresh colour 1's halos.
 * ---------------------------------------------------------------------------------------------- */
typedef struct thrml_lattice thrml_lattice;
/* How a block key becomes the noise of each (spin, chain) is this engine's own definition (the reference never consumes its
 * RngKey: spin_gibbs.rs:61,82-83 draw from the backend's global generator).  Two mappings:
 *   THRML_LATTICE_NOISE_PROGRAM  the explicit program's: the draw of spin n (index inside its colour block) and chain c is
 *       word c & 3 of Philox4x32-10(counter (n, c >> 2, 0, tag), block key); states then equal the explicit program's.
 *   THRML_LATTICE_NOISE_PACKED (the default)  the 32-bit draw is assembled from calls shared as widely as the bit-packed layout
 *       allows: bit b of its top byte is bit n & 31 of word b & 3 of counter (n >> 5, c, 1 + (b >> 2), tag) — two calls give the
 *       top bytes of 32 spins as eight bit planes, compared with the thresholds bit-sliced — and, only when the top byte equals
 *       the threshold's, the low 24 bits of word c & 3 of counter (n, c >> 2, 3, tag).  Same rule (draw <= threshold), same
 *       24-bit resolution, a sixteenth of the generator work per update. */
#define THRML_LATTICE_NOISE_PROGRAM 0
#define THRML_LATTICE_NOISE_PACKED 1
/* The PACKED mapping evaluated spin by spin from the threshold table: the route taken by itself when a threshold's top byte
 * does not depend on the neighbour configuration through the number of up neighbours alone (the bit-sliced comparison needs
 * that); selectable so that tests can run it.  Same noise, same states as PACKED. */
#define THRML_LATTICE_NOISE_PACKED_TABLE 2
int32_t thrml_lattice_set_noise(thrml_lattice* lat, int32_t mapping);
int32_t thrml_lattice_create(thrml_ctx* ctx, int64_t height, int64_t width, int64_t row_begin, int64_t n_rows, float coupling,
                             float bias, float beta, int64_t n_chains, int64_t chain_offset, thrml_lattice** out);
void thrml_lattice_destroy(thrml_lattice* lat);
/* Uniform random spins (asynchronous). */
int32_t thrml_lattice_randomize(thrml_lattice* lat, uint64_t key);
/* Stripe state as bytes 0/1, host layout [chain][stripe row][column]. */
int32_t thrml_lattice_upload(thrml_lattice* lat, const uint8_t* host);
int32_t thrml_lattice_download(thrml_lattice* lat, uint8_t* host);
/* The same state as bits, host layout [chain][stripe row][width / 32] u32, bit k of word v = column 32 v + k: one bit per
 * spin over the host link. */
int32_t thrml_lattice_upload_bits(thrml_lattice* lat, const uint32_t* host);
int32_t thrml_lattice_download_bits(thrml_lattice* lat, uint32_t* host);
/* Update one colour of stripe rows [row_begin, row_end) with the block key (asynchronous).  The other colour's halo
 * rows must be current. */
int32_t thrml_lattice_update(thrml_lattice* lat, int32_t colour, uint64_t block_key, int64_t row_begin, int64_t row_end);
/* Device pointers of the rows a stripe sends (its first and last row of `colour`) and of its two halo rows, and their
 * size: what a multi-process host hands to its point-to-point exchange. */
int32_t thrml_lattice_halo_info(thrml_lattice* lat, int32_t colour, void** send_top, void** send_bottom, void** recv_top,
                                void** recv_bottom, int64_t* row_bytes);
/* Halo refresh between stripes of one process (device-to-device copy), and for a stripe that holds the whole lattice. */
int32_t thrml_lattice_copy_halo(thrml_lattice* dst, int32_t which_dst, const thrml_lattice* src, int32_t which_src, int32_t colour);
int32_t thrml_lattice_wrap_halo(thrml_lattice* lat, int32_t colour);
/* sums_out[2][n_chains] (host, int64): per chain the sum of spins and the sum of s_i s_j over the bonds this stripe owns
 * (each bond is owned by its colour-0 end), from which magnetisation and energy follow. */
int32_t thrml_lattice_observe(thrml_lattice* lat, int64_t* sums_out);
/* The sweep driver inside the library: run_blocks (sampling.rs:81-106) = n_iters sweeps with keys key.split(n_iters), each
 * sweep as described above.  comm = NULL (or a communicator of one rank): the stripe must hold the whole lattice and wraps
 * onto itself.  Otherwise rank r of `comm` holds rows [r H / world, (r + 1) H / world) and the halo rows travel by grouped
 * ncclSend / ncclRecv between ring neighbours: per colour the two boundary rows are updated first and exchanged on a side
 * stream while the interior rows are updated.  record != 0 appends, after every sweep, this stripe's per-chain sum of spins
 * and sum of bond products to a series kept on the device (thrml_lattice_observe's sums, without the host round trip).
 * Asynchronous; collective over `comm`. */
int32_t thrml_lattice_run_blocks(thrml_lattice* lat, uint64_t key, int64_t n_iters, thrml_comm* comm, int32_t record);
/* Both colours' halo rows brought up to date (after an upload or a randomize): wrap, or one exchange per colour. */
int32_t thrml_lattice_refresh_halos(thrml_lattice* lat, thrml_comm* comm);
/* The recorded series, summed over the stripes of `comm` by ONE allreduce: series_out[record][2][chain] (host, int64) =
 * whole-lattice (sum of spins, sum of bond products) after each recorded sweep; n_records_out = records held.  series_out
 * may be NULL to query the count.  thrml_lattice_moments reduces the same series to the first and second moments over the
 * recorded sweeps of m = sum s / N and e = -(J sum_bonds s_i s_j + b sum s) / N: moments_out[4][chain] = <m>, <m^2>, <e>, <e^2>. */
int32_t thrml_lattice_read_series(thrml_lattice* lat, thrml_comm* comm, int64_t* series_out, int64_t capacity_records, int64_t* n_records_out);
int32_t thrml_lattice_moments(thrml_lattice* lat, thrml_comm* comm, double* moments_out, int64_t* n_records_out);
int32_t thrml_lattice_series_reset(thrml_lattice* lat);
int32_t thrml_lattice_synchronize(thrml_lattice* lat);

/* ------------------------------------------------------------------------------------------------
 * Implicit Potts lattice: an nx x ny x nz periodic lattice of categorical nodes (K categories), one K x K table per
 * direction shared by all edges of that direction, per-node unary terms, checkerboard blocks [(x+y+z) even, odd],
 * CategoricalGibbsConditional updates (crates/thrml-samplers/src/softmax.rs:228-271,586-709).  It samples exactly what
 * FactorSamplingProgram (crates/thrml-models/src/factor.rs:153-184) would with the factors
 * CategoricalEBMFactor([nodes], unary[N,K,1]) and CategoricalEBMFactor([u, u+e_d], T_d) for d = x, y, z
 * (crates/thrml-models/src/discrete_ebm.rs:792-851), whose [N,6,K*K] per-block weight tensors never have to exist.
 * tables[3][K][K] (energy term T_d[x_u][x_{u+e_d}]), unary[N][K] (nullable = zeros), node index (x*ny + y)*nz + z.
 * ---------------------------------------------------------------------------------------------- */
typedef struct thrml_potts thrml_potts;
/* Key -> noise mapping of this engine (see thrml_lattice_set_noise for why it is the engine's to define):
 *   THRML_POTTS_NOISE_PROGRAM  the explicit program's: the Gumbel uniform of (node n, chain c, category k) is word k & 3 of
 *       Philox4x32-10(counter (n, c, k >> 2, tag), block key); states then equal the explicit factor program's.
 *   THRML_POTTS_NOISE_QUAD (the default)  word c & 3 of counter (n, c >> 2, k, tag): one call per category serves four chains. */
#define THRML_POTTS_NOISE_PROGRAM 0
#define THRML_POTTS_NOISE_QUAD 1
int32_t thrml_potts_set_noise(thrml_potts* p, int32_t mapping);
int32_t thrml_potts_create(thrml_ctx* ctx, int32_t nx, int32_t ny, int32_t nz, int32_t n_categories, const float* tables,
                           const float* unary, float beta, int64_t n_chains, int64_t chain_offset, thrml_potts** out);
void thrml_potts_destroy(thrml_potts* p);
int32_t thrml_potts_randomize(thrml_potts* p, uint64_t key);
/* Category bytes, host layout [chain][node]. */
int32_t thrml_potts_upload(thrml_potts* p, const uint8_t* host);
int32_t thrml_potts_download(thrml_potts* p, uint8_t* host);
/* Update one colour with its block key (asynchronous); a sweep is colour 0 with key.split(2)[0], then colour 1. */
int32_t thrml_potts_update(thrml_potts* p, int32_t colour, uint64_t block_key);
/* Category-marginal observer: counts[node][category] += chains in that category (asynchronous); read as int32. */
int32_t thrml_potts_observe_marginals(thrml_potts* p);
int32_t thrml_potts_read_marginals(thrml_potts* p, int32_t* counts_out, int64_t* n_obs_out);
/* Zeroes the counts and the observation count (the observer's init, moment.rs:152-172; asynchronous). */
int32_t thrml_potts_reset_marginals(thrml_potts* p);
/* Drivers inside the library: run_blocks (sampling.rs:81-106, asynchronous) and sample_with_observation
 * (sampling.rs:178-320) with the category-marginal observer — warm-up, observe, then n_samples - 1 times
 * (steps_per_sample sweeps, observe).  An observation that follows a sweep is counted by that sweep's update kernels
 * (at most 16 categories, a multiple of 128 chains up to 8064); otherwise by the observer kernel.  With chains sharded over ranks, thrml_potts_marginals_allreduce adds the counts and
 * the observation count over `comm` in place (one grouped ncclAllReduce). */
int32_t thrml_potts_run_blocks(thrml_potts* p, uint64_t key, int64_t n_iters);
int32_t thrml_potts_sample_with_marginals(thrml_potts* p, uint64_t key, int64_t n_warmup, int64_t n_samples, int64_t steps_per_sample);
int32_t thrml_potts_marginals_allreduce(thrml_potts* p, thrml_comm* comm);
int32_t thrml_potts_synchronize(thrml_potts* p);

#ifdef __cplusplus
}
#endif
#endif /* THRML_B200_H */
