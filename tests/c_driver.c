/* A host written in plain C against include/thrml_b200.h alone: the estimate_moments path
 * (crates/thrml-models/src/ising.rs:455-505) on a 16 x 16 periodic Ising lattice, as a compiled host (the reference's own
 * host is compiled code) would call it.  Prints the final states' checksum and the moment sums; the Python test compares
 * them with the oracle.  Usage: c_driver <chains> <key>.  Exit code 0 on success, the library's status otherwise. */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "thrml_b200.h"

#define CHECK(call)                                                                   \
    do {                                                                              \
        int32_t rc_ = (call);                                                         \
        if (rc_ != THRML_OK) {                                                        \
            fprintf(stderr, "%s -> %d: %s\n", #call, (int)rc_, thrml_last_error());   \
            return (int)(-rc_);                                                       \
        }                                                                             \
    } while (0)

int main(int argc, char** argv) {
    const int64_t chains = argc > 1 ? atoll(argv[1]) : 64;
    const uint64_t key = argc > 2 ? strtoull(argv[2], NULL, 10) : 7;
    int64_t side = 0, n_edges = 0;
    CHECK(thrml_lattice_edges(16, 1, &side, &n_edges, NULL, NULL));
    const int64_t n = side * side;
    int64_t* edges = malloc(sizeof(int64_t) * 2 * (size_t)n_edges);
    int32_t* colour = malloc(sizeof(int32_t) * (size_t)n);
    CHECK(thrml_lattice_edges(16, 1, &side, &n_edges, edges, colour));

    int32_t* kinds = calloc((size_t)n, sizeof(int32_t)); /* all spins */
    int64_t* nodes = malloc(sizeof(int64_t) * (size_t)n);
    float* bias = malloc(sizeof(float) * (size_t)n);
    float* J = malloc(sizeof(float) * (size_t)n_edges);
    for (int64_t i = 0; i < n; ++i) {
        nodes[i] = i;
        bias[i] = 0.05f * (float)((i * 37) % 11 - 5); /* any fixed values: the test passes the same ones to the oracle */
    }
    for (int64_t e = 0; e < n_edges; ++e) J[e] = 0.3f + 0.01f * (float)(e % 7);

    thrml_builder* b = NULL;
    const int32_t dtype_order[1] = {0}; /* node_shape_dtypes of an IsingEBM: spins only (ising.rs:145-149) */
    CHECK(thrml_builder_create(kinds, n, dtype_order, 1, &b));
    int64_t* blk[2];
    int64_t len[2] = {0, 0};
    for (int c = 0; c < 2; ++c) blk[c] = malloc(sizeof(int64_t) * (size_t)n);
    for (int64_t i = 0; i < n; ++i) blk[colour[i]][len[colour[i]]++] = i;
    for (int c = 0; c < 2; ++c) CHECK(thrml_builder_add_free_block(b, blk[c], len[c], c, THRML_SAMPLER_SPIN_GIBBS));
    CHECK(thrml_builder_add_ising(b, nodes, n, bias, edges, n_edges, J, 1.0f));
    CHECK(thrml_builder_compile(b));

    thrml_ctx* ctx = NULL;
    thrml_program* prog = NULL;
    thrml_state* st = NULL;
    thrml_moments* mom = NULL;
    CHECK(thrml_ctx_create(0, &ctx));
    CHECK(thrml_program_create(ctx, b, &prog));
    CHECK(thrml_state_create(prog, chains, 0, &st));

    /* hinton_init (ising.rs:602-673): biases gathered block by block */
    float* gathered = malloc(sizeof(float) * (size_t)n);
    int64_t at = 0;
    for (int c = 0; c < 2; ++c)
        for (int64_t i = 0; i < len[c]; ++i) gathered[at++] = bias[blk[c][i]];
    const int32_t both[2] = {0, 1};
    CHECK(thrml_hinton_init(st, both, 2, gathered, 1.0f, key, NULL));

    /* MomentAccumulatorObserver::ising_moment_spec (moment.rs:125-148): all nodes, all edges */
    const int64_t rows_per_type[2] = {n, n_edges};
    int64_t* row_ptr = malloc(sizeof(int64_t) * (size_t)(n + n_edges + 1));
    int64_t* members = malloc(sizeof(int64_t) * (size_t)(n + 2 * n_edges));
    for (int64_t i = 0; i <= n; ++i) row_ptr[i] = i;
    for (int64_t e = 1; e <= n_edges; ++e) row_ptr[n + e] = n + 2 * e;
    for (int64_t i = 0; i < n; ++i) members[i] = i;
    for (int64_t e = 0; e < 2 * n_edges; ++e) members[n + e] = edges[e];
    CHECK(thrml_moments_create(prog, 2, rows_per_type, row_ptr, members, 1, &mom));
    CHECK(thrml_sample_with_observation(st, key + 1, 20, 31, 2, mom, NULL, 0, NULL, NULL));

    uint64_t checksum = 1469598103934665603ull; /* FNV-1a over the final states, block by block, [chain][node] */
    for (int c = 0; c < 2; ++c) {
        uint8_t* host = malloc((size_t)(len[c] * chains));
        CHECK(thrml_state_download_u8(st, c, host));
        for (int64_t i = 0; i < len[c] * chains; ++i) checksum = (checksum ^ host[i]) * 1099511628211ull;
        free(host);
    }
    int64_t* s1 = malloc(sizeof(int64_t) * (size_t)n);
    int64_t* s2 = malloc(sizeof(int64_t) * (size_t)n_edges);
    int64_t n_obs = 0;
    CHECK(thrml_moments_read(mom, 0, s1, &n_obs));
    CHECK(thrml_moments_read(mom, 1, s2, &n_obs));
    int64_t t1 = 0, t2 = 0, w1 = 0, w2 = 0;
    for (int64_t i = 0; i < n; ++i) { t1 += s1[i]; w1 += (i + 1) * s1[i]; }
    for (int64_t e = 0; e < n_edges; ++e) { t2 += s2[e]; w2 += (e + 1) * s2[e]; }
    printf("%llu %lld %lld %lld %lld %lld\n", (unsigned long long)checksum, (long long)n_obs, (long long)t1, (long long)w1, (long long)t2, (long long)w2);

    thrml_moments_destroy(mom);
    thrml_state_destroy(st);
    thrml_program_destroy(prog);
    thrml_ctx_destroy(ctx);
    thrml_builder_destroy(b);
    return 0;
}
