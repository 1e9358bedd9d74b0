/*
 * CPU oracle, C form: the same migration and swap semantics as kv_oracle.py,
 * stated with pointers and strides, one memcpy per contiguous run, OpenMP over
 * (block, layer).  TEST INFRASTRUCTURE ONLY: built by oracle/build_oracle.py
 * into oracle/_build/, loaded by oracle/kv_oracle_c.py, used by the tests as a
 * second checker and by the benchmark as a timed CPU arm.  PARITY UNPINNED: see
 * kv_oracle.py for what the restatement rests on.
 *
 * Pool layout [num_blocks, layers_local, heads_local, block_size, head_dim],
 * K and V separately (distserve/worker.py:107-121); a worker (tp, t, pp, p)
 * holds layers [p*L/pp, (p+1)*L/pp) and heads [t*H/tp, (t+1)*H/tp)
 * (distserve/config.py:244-257,279-286).
 */
#include <stdint.h>
#include <string.h>

/*
 * ctx_k / ctx_v: ctx_pp*ctx_tp pool base pointers indexed [pp_rank*ctx_tp + tp_rank]
 * (NULL allowed for workers that do not contribute).  Returns 0, or -1 on a bad
 * argument (lengths, divisibility), having written nothing.
 */
int kv_oracle_migrate(const uint8_t* const* ctx_k, const uint8_t* const* ctx_v,
                      int64_t ctx_tp, int64_t ctx_pp,
                      const int64_t* ctx_blocks, int64_t n_ctx,
                      int64_t dec_tp, int64_t dec_tp_rank, int64_t dec_pp, int64_t dec_pp_rank,
                      const int64_t* dec_blocks, int64_t n_dec,
                      uint8_t* k_cache, uint8_t* v_cache,
                      int64_t num_layers, int64_t num_heads, int64_t slab_bytes /* block_size*head_dim*elem */)
{
    if (n_ctx != n_dec || n_ctx < 0) return -1;
    if (ctx_tp <= 0 || ctx_pp <= 0 || dec_tp <= 0 || dec_pp <= 0) return -1;
    /* Multi-query attention: the one KV head is held by every tensor-parallel rank of either stage
     * (distserve/config.py:233-237); a decoding rank reads the replica at the matching position. */
    const int replicated = num_heads == 1;
    if (num_layers % ctx_pp || num_layers % dec_pp) return -1;
    if (!replicated && (num_heads % ctx_tp || num_heads % dec_tp)) return -1;
    const int64_t Ld = num_layers / dec_pp, Hd = replicated ? 1 : num_heads / dec_tp;
    const int64_t Lc = num_layers / ctx_pp, Hc = replicated ? 1 : num_heads / ctx_tp;
    const int64_t dst_block = Ld * Hd * slab_bytes, src_block = Lc * Hc * slab_bytes;

#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t i = 0; i < n_ctx; ++i) {
        for (int64_t dl = 0; dl < Ld; ++dl) {
            const int64_t gl = dec_pp_rank * Ld + dl;          /* global layer */
            const int64_t cp = gl / Lc, cl = gl % Lc;          /* owning pipeline rank, its local layer */
            int64_t dh = 0;
            while (dh < Hd) {
                const int64_t gh = replicated ? 0 : dec_tp_rank * Hd + dh;      /* global head */
                const int64_t ct = replicated ? dec_tp_rank * ctx_tp / dec_tp : gh / Hc;   /* owning (or replica) tensor rank */
                const int64_t ch = gh % Hc;                                       /* its local head */
                int64_t run = Hc - ch;                         /* heads left in that owner's chunk ... */
                if (run > Hd - dh) run = Hd - dh;              /* ... and in this worker's range */
                const int64_t w = cp * ctx_tp + ct;
                const size_t soff = (size_t)(ctx_blocks[i] * src_block + (cl * Hc + ch) * slab_bytes);
                const size_t doff = (size_t)(dec_blocks[i] * dst_block + (dl * Hd + dh) * slab_bytes);
                memcpy(k_cache + doff, ctx_k[w] + soff, (size_t)(run * slab_bytes));
                memcpy(v_cache + doff, ctx_v[w] + soff, (size_t)(run * slab_bytes));
                dh += run;
            }
        }
    }
    return 0;
}

/* Block swap in list order (distserve/worker.py:269-311); sequential so that a repeated target keeps the last source. */
int kv_oracle_swap(const int64_t* source_ids, int64_t n_source, const int64_t* target_ids, int64_t n_target, int is_swap_in,
                   uint8_t* k_cache, uint8_t* v_cache, uint8_t* k_swap, uint8_t* v_swap, int64_t block_bytes)
{
    if (n_source != n_target || n_source < 0) return -1;
    for (int64_t i = 0; i < n_source; ++i) {
        const size_t s = (size_t)(source_ids[i] * block_bytes), t = (size_t)(target_ids[i] * block_bytes);
        if (is_swap_in) {
            memcpy(k_cache + t, k_swap + s, (size_t)block_bytes);
            memcpy(v_cache + t, v_swap + s, (size_t)block_bytes);
        } else {
            memcpy(k_swap + t, k_cache + s, (size_t)block_bytes);
            memcpy(v_swap + t, v_cache + s, (size_t)block_bytes);
        }
    }
    return 0;
}
