// Index arithmetic of the column-sharded products (host only, no CUDA): which columns a rank owns,
// and how the rows of A are cut into the chunks that the host-buffer pipeline uploads and gathers.
// Kept apart from the CUDA sources so that the CPU tests can pin it through the C ABI
// (b200_shard_columns, b200_shard_host_plan) against its Python mirror.
#pragma once

#include <cstdint>

#include "../../include/b200_gemm.h"

namespace b200_shard {

constexpr int64_t kColumnAlign = 32;  // shard boundaries fall on 128-byte column groups: TMA- and vector-store-legal

// Columns [col0, col0 + cols) of rank `rank`: equal blocks rounded up to kColumnAlign columns, the
// last ranks taking what is left (possibly nothing when N is small).
inline void columns(int64_t N, int world, int rank, int64_t* col0, int64_t* cols) {
    int64_t per = (N + world - 1) / world;
    per = (per + kColumnAlign - 1) / kColumnAlign * kColumnAlign;
    const int64_t c0 = per * rank < N ? per * rank : N;
    const int64_t c1 = c0 + per < N ? c0 + per : N;
    *col0 = c0;
    *cols = c1 - c0;
}

// Rank r holds the contiguous rows [r * rows_per_rank, (r + 1) * rows_per_rank) of A on its host and
// uploads them in `chunks` pieces of chunk_rows rows.  Chunk ch of every rank is gathered into one
// block of world * chunk_rows rows (rank-major), which is multiplied as one strip; row i of rank r's
// piece of strip ch is global row r * rows_per_rank + ch * chunk_rows + i.
// chunks <= 0 picks: 4 pieces when the rows divide, else 2, else 1.
inline bool host_plan(int64_t M, int world, int chunks, b200_shard_host_layout* out) {
    if (M <= 0 || world < 1 || M % world != 0 || chunks > B200_SHARD_MAX_CHUNKS) return false;
    const int64_t per = M / world;
    if (chunks <= 0) chunks = (per % 4 == 0 && per >= 512) ? 4 : (per % 2 == 0 && per >= 256) ? 2 : 1;
    if (per % chunks != 0) return false;
    out->chunks = chunks;
    out->rows_per_rank = per;
    out->chunk_rows = per / chunks;
    return true;
}

}  // namespace b200_shard
