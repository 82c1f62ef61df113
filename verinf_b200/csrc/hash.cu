// BLAKE3 column hashing, Merkle levels, pad PRG and challenge PRF for sm_100a.
//
// Replaces prover/kernels/blake3_columns.cuh (k_hash_columns_simple, k_stream_*),
// prover/kernels/merkle.cuh (k_level), k_row_prg(_indexed) and k_challenge_vec/_at
// (prover/cuda_primitives.py:566-591,796-1004).
//
// Column hash design: all columns advance in lockstep, so the BLAKE3 chunk counter
// and the shape of the chaining-value stack are the same for every column and live
// on the host.  The device state is only the stack contents, indexed by subtree
// size instead of by a stack pointer: level b holds the chaining value of a
// complete subtree of 2^b chunks (the binary-counter form of BLAKE3's incremental
// tree), stored [level][word][column] so every access is coalesced.
#include <cstdlib>
#include <mutex>

#include "../../include/verinf_b200.h"
#include "blake3.cuh"
#include "common.cuh"
#include "gl.cuh"

namespace {

constexpr int CHUNK_ROWS = 128;   // 1024-byte BLAKE3 chunk = 128 field elements

struct StreamArgs {
    const uint64_t* rows;   // first row of this call, row-major, leading dimension ncols
    int64_t ncols;
    int64_t n_rows;         // rows in this call
    uint64_t count0;        // chunks hashed before this call
    uint64_t ctr_base;      // added to the chunk index to form the BLAKE3 chunk counter (sub-tree hashing)
    uint64_t total_chunks;  // chunks of the whole stream (>= 1)
    uint32_t* state;        // [level][8][ncols]
    uint32_t* digests;      // (ncols, 8) words; written by the call that ends the stream
    // segmented mode (gridDim.y > 1): segment y hashes rows [y*seg_rows, ...) as its own non-final
    // stream with chunk counters offset by y*seg_rows/128 and its own state block
    int64_t seg_rows;       // rows per segment (multiple of 128), 0 = not segmented
    int64_t seg_state;      // uint32 words of state per segment
};

__global__ void __launch_bounds__(128) k_hash_stream(StreamArgs a) {
    const int64_t col = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= a.ncols) return;
    const int64_t ld = a.ncols;
    if (a.seg_rows) {        // this CTA row works on one segment
        const int64_t seg = blockIdx.y;
        a.rows += seg * a.seg_rows * ld;
        a.n_rows = a.n_rows - seg * a.seg_rows < a.seg_rows ? a.n_rows - seg * a.seg_rows : a.seg_rows;
        a.ctr_base += (uint64_t)(seg * (a.seg_rows / CHUNK_ROWS));
        a.state += seg * a.seg_state;
    }
    const uint64_t* p = a.rows + col;
    const int64_t n_chunks = a.n_rows == 0 ? 1 : (a.n_rows + CHUNK_ROWS - 1) / CHUNK_ROWS;
    const bool single = a.total_chunks == 1;

    for (int64_t ch = 0; ch < n_chunks; ++ch) {
        const uint64_t count = a.count0 + (uint64_t)ch;           // = this chunk's counter
        int64_t r0 = ch * CHUNK_ROWS;
        int64_t rows_here = a.n_rows - r0 < CHUNK_ROWS ? a.n_rows - r0 : CHUNK_ROWS;
        int nb = rows_here == 0 ? 1 : (int)((rows_here + 7) / 8);
        uint32_t cv[8];
        vb3::set_iv(cv);
        if (rows_here == CHUNK_ROWS) {
            // whole chunk: 16 full blocks, no row guards, constant block length (4.52 -> 4.18 ms for the
            // 4096 x 2^18 matrix against the guarded loop below)
            const uint64_t* q = p + r0 * ld;
#pragma unroll 1
            for (int b = 0; b < 16; ++b) {
                uint32_t m[16];
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    const uint64_t x = __ldg(q + r * ld);
                    m[2 * r] = (uint32_t)x;
                    m[2 * r + 1] = (uint32_t)(x >> 32);
                }
                q += 8 * ld;
                const uint32_t flags = (b == 0 ? vb3::CHUNK_START : 0) |
                                       (b == 15 ? (vb3::CHUNK_END | (single ? vb3::ROOT : 0)) : 0);
                vb3::compress(cv, m, a.ctr_base + count, 64, flags);
            }
        } else
        for (int b = 0; b < nb; ++b) {
            int64_t rb = rows_here - b * 8 < 8 ? rows_here - b * 8 : 8;
            uint32_t m[16];
            const uint64_t* q = p + (r0 + b * 8) * ld;
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                uint64_t x = r < rb ? __ldg(q + r * ld) : 0;
                m[2 * r] = (uint32_t)x;
                m[2 * r + 1] = (uint32_t)(x >> 32);
            }
            uint32_t flags = (b == 0 ? vb3::CHUNK_START : 0) |
                             (b == nb - 1 ? (vb3::CHUNK_END | (single ? vb3::ROOT : 0)) : 0);
            vb3::compress(cv, m, a.ctr_base + count, (uint32_t)(rb * 8), flags);
        }
        const bool is_final = count + 1 == a.total_chunks;
        if (!is_final) {
            // binary-counter carry: merge with every complete subtree whose bit is set
            int b = 0;
            while ((count >> b) & 1) {
                uint32_t l[8], o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) l[i] = a.state[((int64_t)b * 8 + i) * a.ncols + col];
                vb3::parent(l, cv, 0, o);
#pragma unroll
                for (int i = 0; i < 8; ++i) cv[i] = o[i];
                ++b;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) a.state[((int64_t)b * 8 + i) * a.ncols + col] = cv[i];
        } else {
            // close the tree: fold in the pending subtrees, smallest first; the last merge is the root
            uint64_t rem = count;
            int b = 0;
            while (rem) {
                if (rem & 1) {
                    uint32_t l[8], o[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) l[i] = a.state[((int64_t)b * 8 + i) * a.ncols + col];
                    vb3::parent(l, cv, (rem >> 1) == 0 ? vb3::ROOT : 0, o);
#pragma unroll
                    for (int i = 0; i < 8; ++i) cv[i] = o[i];
                }
                rem >>= 1;
                ++b;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) a.digests[col * 8 + i] = cv[i];
        }
    }
}

__global__ void __launch_bounds__(128) k_merkle_level(const uint32_t* __restrict__ in, int64_t n_in,
                                                      uint32_t* __restrict__ out, int64_t n_out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_out) return;
    const int64_t li = 2 * i, ri = (2 * i + 1 < n_in) ? 2 * i + 1 : 2 * i;
    uint32_t m[16], h[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) { m[k] = __ldg(in + li * 8 + k); m[8 + k] = __ldg(in + ri * 8 + k); }
    vb3::hash_one_block(m, 64, h);
#pragma unroll
    for (int k = 0; k < 8; ++k) out[i * 8 + k] = h[k];
}

// All levels above a level of at most MERKLE_TOP_NODES nodes in one single-CTA launch (a level per
// loop iteration, block barrier in between) instead of one launch per level: the upper eleven
// levels of a tree are launch latency only.  Loads are plain (not read-only-cache) loads because
// each level reads what the previous iteration of the same kernel wrote.
constexpr int MERKLE_TOP_NODES = 2048;
__global__ void __launch_bounds__(512) k_merkle_top(const uint32_t* in, int64_t n_in, uint32_t* out) {
    const uint32_t* cur = in;
    uint32_t* nxt = out;
    int64_t n = n_in;
    while (n > 1) {
        const int64_t n_out = (n + 1) >> 1;
        for (int64_t i = threadIdx.x; i < n_out; i += blockDim.x) {
            const int64_t li = 2 * i, ri = (2 * i + 1 < n) ? 2 * i + 1 : 2 * i;
            uint32_t m[16], h[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) { m[k] = cur[li * 8 + k]; m[8 + k] = cur[ri * 8 + k]; }
            vb3::hash_one_block(m, 64, h);
#pragma unroll
            for (int k = 0; k < 8; ++k) nxt[i * 8 + k] = h[k];
        }
        __syncthreads();
        cur = nxt;
        nxt += n_out * 8;
        n = n_out;
    }
}

__global__ void __launch_bounds__(256) k_row_prg(const uint8_t* __restrict__ seed, int64_t row_off,
                                                 const uint64_t* __restrict__ rows, int64_t n_rows,
                                                 int64_t slack, uint64_t* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * slack) return;
    const int64_t r = i / slack, k = i - r * slack;
    uint32_t s[8];
    vb3::load_seed(seed, s);
    const uint64_t row = rows ? rows[r] : (uint64_t)(row_off + r);
    out[i] = vb3::pad_prg(s, row, (uint64_t)k);
}

__global__ void __launch_bounds__(256) k_challenge(const uint8_t* __restrict__ seed,
                                                   const uint8_t* __restrict__ label, int label_len,
                                                   const uint64_t* __restrict__ cids, int64_t n,
                                                   uint64_t* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    uint32_t s[8];
    vb3::load_seed(seed, s);
    out[i] = vb3::challenge(s, vb3::load_label(label, label_len), label_len, cids ? cids[i] : (uint64_t)i);
}

// state level -> (ncols, 8 words) rows
__global__ void __launch_bounds__(128) k_state_level_out(const uint32_t* __restrict__ state, int level,
                                                         int64_t ncols, uint32_t* __restrict__ out) {
    const int64_t col = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= ncols) return;
#pragma unroll
    for (int i = 0; i < 8; ++i) out[col * 8 + i] = state[((int64_t)level * 8 + i) * ncols + col];
}

// Merge sub-tree chaining values into column digests.  The merge order depends only on the block
// sizes, which are the same for every column, so the host compiles it into a short program:
// op 0 = push the next block, op 1 = merge the two top entries, op 2 = merge them as the root.
constexpr int MAX_MERGE_OPS = 192, MAX_MERGE_DEPTH = 48;
struct MergeArgs {
    const uint32_t* cvs;   // (nblocks, ncols, 8 words)
    int64_t ncols;
    int n_ops;
    unsigned char ops[MAX_MERGE_OPS];
    uint32_t* digests;
};
__global__ void __launch_bounds__(128) k_merge_subtrees(MergeArgs a) {
    const int64_t col = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= a.ncols) return;
    uint32_t st[MAX_MERGE_DEPTH][8];
    int sp = 0, next = 0;
    for (int o = 0; o < a.n_ops; ++o) {
        if (a.ops[o] == 0) {
            const uint32_t* src = a.cvs + ((int64_t)next * a.ncols + col) * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) st[sp][i] = __ldg(src + i);
            ++sp; ++next;
        } else {
            uint32_t l[8], r[8], out[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) { l[i] = st[sp - 2][i]; r[i] = st[sp - 1][i]; }
            vb3::parent(l, r, a.ops[o] == 2 ? vb3::ROOT : 0, out);
            --sp;
#pragma unroll
            for (int i = 0; i < 8; ++i) st[sp - 1][i] = out[i];
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) a.digests[col * 8 + i] = st[0][i];
}

// gather the sub-tree values a segmented run left in the per-segment states into (nblocks, ncols, 8)
constexpr int MAX_SEG_BLOCKS = 96;
struct GatherArgs {
    const uint32_t* state;
    int64_t seg_state, ncols;
    int nblocks;
    unsigned char seg[MAX_SEG_BLOCKS], level[MAX_SEG_BLOCKS];
    uint32_t* cvs;
};
__global__ void __launch_bounds__(128) k_gather_blocks(GatherArgs a) {
    const int64_t col = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    if (col >= a.ncols) return;
    const uint32_t* st = a.state + (int64_t)a.seg[b] * a.seg_state + (int64_t)a.level[b] * 8 * a.ncols + col;
    uint32_t* dst = a.cvs + ((int64_t)b * a.ncols + col) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) dst[i] = st[(int64_t)i * a.ncols];
}

int state_levels(int64_t total_chunks) {
    int b = 1;
    while ((int64_t(1) << b) < total_chunks) ++b;
    return b + 1;
}

}  // namespace

extern "C" int64_t vi_hash_stream_state_bytes(int64_t ncols, int64_t total_rows) {
    if (ncols <= 0) return 0;
    int64_t chunks = total_rows <= 0 ? 1 : (total_rows + CHUNK_ROWS - 1) / CHUNK_ROWS;
    return (int64_t)state_levels(chunks) * 32 * ncols;
}

extern "C" int vi_hash_stream_update(void* state, int64_t ncols, int64_t total_rows, int64_t rows_done,
                                     const uint64_t* rows, int64_t n_rows, uint8_t* digests, void* stream) {
    VI_REQUIRE(ncols >= 0 && total_rows >= 0 && rows_done >= 0 && n_rows >= 0, "hash stream: negative size");
    VI_REQUIRE(rows_done + n_rows <= total_rows, "hash stream: more rows than announced (%lld + %lld > %lld)",
               (long long)rows_done, (long long)n_rows, (long long)total_rows);
    VI_REQUIRE(rows_done % CHUNK_ROWS == 0, "hash stream: rows_done must be a multiple of 128");
    const bool ends = rows_done + n_rows == total_rows;
    VI_REQUIRE(ends || n_rows % CHUNK_ROWS == 0, "hash stream: only the last call may bring a partial chunk");
    if (ncols == 0) return VI_OK;
    if (n_rows == 0 && !(ends && total_rows == 0)) return VI_OK;
    VI_REQUIRE(state != nullptr, "hash stream: null state");
    VI_REQUIRE(!ends || digests != nullptr, "hash stream: the closing call needs a digest buffer");
    VI_REQUIRE(n_rows == 0 || rows != nullptr, "hash stream: null rows");
    StreamArgs a;
    a.rows = rows; a.ncols = ncols; a.n_rows = n_rows;
    a.count0 = (uint64_t)(rows_done / CHUNK_ROWS);
    a.ctr_base = 0; a.seg_rows = 0; a.seg_state = 0;
    a.total_chunks = total_rows == 0 ? 1 : (uint64_t)((total_rows + CHUNK_ROWS - 1) / CHUNK_ROWS);
    a.state = (uint32_t*)state; a.digests = (uint32_t*)digests;
    const int block = 128;
    vi::ProfScope prof(vi::PROF_HASH, (cudaStream_t)stream);
    k_hash_stream<<<(unsigned)((ncols + block - 1) / block), block, 0, (cudaStream_t)stream>>>(a);
    return vi::check_launch("k_hash_stream");
}

extern "C" int64_t vi_hash_subtree_state_bytes(int64_t ncols, int level) {
    if (level < 0 || level > 40) return 0;
    return vi_hash_stream_state_bytes(ncols, ((int64_t(1) << level) + 1) * CHUNK_ROWS);
}

extern "C" int vi_hash_subtree(const uint64_t* rows, int64_t n_rows, int64_t ncols, int64_t first_chunk, int level,
                               void* state, uint8_t* cv_out, void* stream) {
    VI_REQUIRE(level >= 0 && level <= 40, "hash_subtree: level out of range");
    VI_REQUIRE(ncols >= 0 && first_chunk >= 0, "hash_subtree: negative size");
    const int64_t chunks = int64_t(1) << level;
    VI_REQUIRE(n_rows > (chunks - 1) * CHUNK_ROWS && n_rows <= chunks * CHUNK_ROWS,
               "hash_subtree: %lld rows are not 2^%d chunks of 128 rows (only the last chunk may be short)",
               (long long)n_rows, level);
    VI_REQUIRE(first_chunk % chunks == 0, "hash_subtree: first_chunk must be a multiple of 2^level");
    if (ncols == 0) return VI_OK;
    VI_REQUIRE(rows && state && cv_out, "hash_subtree: null pointer");
    StreamArgs a;
    a.rows = rows; a.ncols = ncols; a.n_rows = n_rows;
    a.count0 = 0; a.ctr_base = (uint64_t)first_chunk;
    a.total_chunks = (uint64_t)chunks + 1;            // never final: no ROOT inside a sub-tree
    a.state = (uint32_t*)state; a.digests = nullptr; a.seg_rows = 0; a.seg_state = 0;
    const int block = 128;
    const unsigned grid = (unsigned)((ncols + block - 1) / block);
    {
        vi::ProfScope prof(vi::PROF_HASH, (cudaStream_t)stream);
        k_hash_stream<<<grid, block, 0, (cudaStream_t)stream>>>(a);
    }
    k_state_level_out<<<grid, block, 0, (cudaStream_t)stream>>>((const uint32_t*)state, level, ncols, (uint32_t*)cv_out);
    return vi::check_launch("k_hash_stream<subtree>");
}

extern "C" int vi_hash_merge_subtrees(const uint8_t* cvs, const int32_t* levels, int nblocks, int64_t ncols,
                                      uint8_t* digests, void* stream) {
    VI_REQUIRE(nblocks >= 2, "hash_merge: at least two sub-trees are needed (a single one would need the root flag inside)");
    VI_REQUIRE(ncols >= 0 && levels, "hash_merge: bad arguments");
    MergeArgs a;
    a.cvs = (const uint32_t*)cvs; a.ncols = ncols; a.digests = (uint32_t*)digests; a.n_ops = 0;
    // binary-counter merging of equal-sized neighbours, the last block is not merged eagerly,
    // then a right-to-left fold whose last merge is the root (BLAKE3's incremental tree)
    int stack[MAX_MERGE_DEPTH], sp = 0;
    auto emit = [&](unsigned char op) { if (a.n_ops < MAX_MERGE_OPS) a.ops[a.n_ops] = op; ++a.n_ops; };
    for (int i = 0; i < nblocks; ++i) {
        VI_REQUIRE(levels[i] >= 0 && levels[i] <= 40, "hash_merge: bad level");
        VI_REQUIRE(sp == 0 || stack[sp - 1] >= levels[i], "hash_merge: blocks are not a left-to-right decomposition");
        VI_REQUIRE(sp < MAX_MERGE_DEPTH, "hash_merge: too many pending sub-trees");
        stack[sp++] = levels[i];
        emit(0);
        if (i == nblocks - 1) break;
        while (sp >= 2 && stack[sp - 1] == stack[sp - 2]) { --sp; ++stack[sp - 1]; emit(1); }
    }
    while (sp >= 2) { --sp; emit(sp == 1 ? 2 : 1); }
    VI_REQUIRE(a.n_ops <= MAX_MERGE_OPS, "hash_merge: merge program too long (%d ops)", a.n_ops);
    if (ncols == 0) return VI_OK;
    VI_REQUIRE(cvs && digests, "hash_merge: null pointer");
    const int block = 128;
    k_merge_subtrees<<<(unsigned)((ncols + block - 1) / block), block, 0, (cudaStream_t)stream>>>(a);
    return vi::check_launch("k_merge_subtrees");
}

namespace {
// Row segmentation of a one-shot column hash: with few columns one thread per column leaves the
// GPU empty, so the rows are cut into up to 64 segments of 2^seg_level chunks that are hashed
// concurrently (grid.y) to sub-tree values and then folded.  seg_level < 0: not worth it.
struct SegPlan { int seg_level; int64_t nseg, seg_rows, seg_state_words, state_bytes, cvs_bytes; int nblocks; };
SegPlan seg_plan(int64_t m, int64_t ncols) {
    SegPlan p{-1, 0, 0, 0, 0, 0, 0};
    const int64_t chunks = (m + CHUNK_ROWS - 1) / CHUNK_ROWS;
    // From 131072 columns up one thread per column fills the GPU (at 2^18 columns 8 segments made the hash
    // kernel 6 % faster but the commit only 0.5 %, for 0.3 GB more scratch).
    if (ncols <= 0 || chunks < 4 || ncols >= 131072) return p;
    int64_t want = (262144 + ncols - 1) / ncols;                          // segments that would fill the GPU
    if (want > 64) want = 64;
    int lvl = 0;
    while ((chunks >> (lvl + 1)) >= want) ++lvl;             // largest 2^lvl with chunks / 2^lvl >= want
    int64_t nseg = (chunks + (int64_t(1) << lvl) - 1) >> lvl;
    while (nseg > 64) { ++lvl; nseg = (chunks + (int64_t(1) << lvl) - 1) >> lvl; }
    if (nseg < 2) return p;
    p.seg_level = lvl; p.nseg = nseg; p.seg_rows = (int64_t(1) << lvl) * CHUNK_ROWS;
    p.seg_state_words = (int64_t)(lvl + 2) * 8 * ncols;
    p.state_bytes = p.seg_state_words * 4 * nseg;
    const int64_t tail = chunks - (nseg - 1) * (int64_t(1) << lvl);      // chunks of the last segment
    p.nblocks = (int)(nseg - 1) + __builtin_popcountll((unsigned long long)tail);
    p.cvs_bytes = (int64_t)p.nblocks * ncols * 32;
    return p;
}
}  // namespace

extern "C" int64_t vi_hash_columns_scratch_bytes(int64_t m, int64_t ncols) {
    SegPlan p = seg_plan(m, ncols);
    if (p.seg_level >= 0) return p.state_bytes + p.cvs_bytes;
    return vi_hash_stream_state_bytes(ncols, m);
}

extern "C" int vi_hash_columns(const uint64_t* mat, int64_t m, int64_t ncols, uint8_t* digests,
                               void* scratch, int64_t scratch_bytes, void* stream) {
    VI_REQUIRE(m >= 0 && ncols >= 0, "hash_columns: negative size");
    if (ncols == 0) return VI_OK;
    const SegPlan sp = seg_plan(m, ncols);
    if (sp.seg_level >= 0 && scratch != nullptr && scratch_bytes >= sp.state_bytes + sp.cvs_bytes) {
        cudaStream_t st = (cudaStream_t)stream;
        VI_REQUIRE(mat && digests, "hash_columns: null pointer");
        StreamArgs a;
        a.rows = mat; a.ncols = ncols; a.n_rows = m; a.count0 = 0; a.ctr_base = 0;
        a.total_chunks = (uint64_t(1) << sp.seg_level) + 1;          // segments never close the tree
        a.state = (uint32_t*)scratch; a.digests = nullptr;
        a.seg_rows = sp.seg_rows; a.seg_state = sp.seg_state_words;
        const int block = 128;
        dim3 grid((unsigned)((ncols + block - 1) / block), (unsigned)sp.nseg);
        {
            vi::ProfScope prof(vi::PROF_HASH, st);
            k_hash_stream<<<grid, block, 0, st>>>(a);
        }
        // blocks left to right: full segments at seg_level, then the binary decomposition of the tail
        GatherArgs g;
        int32_t levels[MAX_SEG_BLOCKS];
        g.state = (const uint32_t*)scratch; g.seg_state = sp.seg_state_words; g.ncols = ncols; g.nblocks = 0;
        g.cvs = (uint32_t*)((char*)scratch + sp.state_bytes);
        const int64_t chunks = (m + CHUNK_ROWS - 1) / CHUNK_ROWS;
        const int64_t tail = chunks - (sp.nseg - 1) * (int64_t(1) << sp.seg_level);
        for (int64_t sgi = 0; sgi < sp.nseg - 1; ++sgi) {
            g.seg[g.nblocks] = (unsigned char)sgi; g.level[g.nblocks] = (unsigned char)sp.seg_level;
            levels[g.nblocks++] = sp.seg_level;
        }
        for (int b = 40; b >= 0; --b)
            if ((tail >> b) & 1) {
                g.seg[g.nblocks] = (unsigned char)(sp.nseg - 1); g.level[g.nblocks] = (unsigned char)b;
                levels[g.nblocks++] = b;
            }
        dim3 ggrid(grid.x, (unsigned)g.nblocks);
        k_gather_blocks<<<ggrid, block, 0, st>>>(g);
        int rc = vi::check_launch("k_hash_stream<segments>");
        if (rc) return rc;
        return vi_hash_merge_subtrees((const uint8_t*)g.cvs, levels, g.nblocks, ncols, digests, stream);
    }
    int64_t need = vi_hash_stream_state_bytes(ncols, m);
    if (m > CHUNK_ROWS && (scratch == nullptr || scratch_bytes < need))
        return vi::fail(VI_ERR_SCRATCH, "hash_columns: scratch of %lld bytes required", (long long)need);
    // a single-chunk input never touches the state
    void* st = m > CHUNK_ROWS ? scratch : (void*)digests;
    return vi_hash_stream_update(st, ncols, m, 0, mat, m, digests, stream);
}

extern "C" int64_t vi_merkle_upper_nodes(int64_t n) {
    int64_t t = 0;
    while (n > 1) { n = (n + 1) / 2; t += n; }
    return t;
}

extern "C" int vi_merkle_level(const uint8_t* nodes, int64_t n_nodes, uint8_t* parents, void* stream) {
    VI_REQUIRE(n_nodes >= 0, "merkle: negative size");
    if (n_nodes <= 1) return VI_OK;
    VI_REQUIRE(nodes && parents, "merkle: null pointer");
    VI_REQUIRE(((uintptr_t)nodes & 3) == 0 && ((uintptr_t)parents & 3) == 0, "merkle: buffers must be 4-byte aligned");
    int64_t n_out = (n_nodes + 1) / 2;
    const int block = 128;
    vi::ProfScope prof(vi::PROF_MERKLE, (cudaStream_t)stream);
    k_merkle_level<<<(unsigned)((n_out + block - 1) / block), block, 0, (cudaStream_t)stream>>>(
        (const uint32_t*)nodes, n_nodes, (uint32_t*)parents, n_out);
    return vi::check_launch("k_merkle_level");
}

extern "C" int vi_merkle_build(const uint8_t* leaves, int64_t n, uint8_t* upper, void* stream) {
    VI_REQUIRE(n >= 0, "merkle: negative size");
    const uint8_t* cur = leaves;
    uint8_t* nxt = upper;
    while (n > MERKLE_TOP_NODES) {
        int rc = vi_merkle_level(cur, n, nxt, stream);
        if (rc) return rc;
        n = (n + 1) / 2;
        cur = nxt;
        nxt += n * 32;
    }
    if (n > 1) {
        VI_REQUIRE(cur != nullptr && nxt != nullptr, "merkle: null pointer");
        vi::ProfScope prof(vi::PROF_MERKLE, (cudaStream_t)stream);
        k_merkle_top<<<1, 512, 0, (cudaStream_t)stream>>>((const uint32_t*)cur, n, (uint32_t*)nxt);
        return vi::check_launch("k_merkle_top");
    }
    return VI_OK;
}

extern "C" int vi_row_prg(const uint8_t* seed_dev, int64_t row_off, const uint64_t* rows_dev,
                          int64_t n_rows, int64_t slack, uint64_t* out, void* stream) {
    VI_REQUIRE(n_rows >= 0 && slack >= 0, "row_prg: negative size");
    if (n_rows == 0 || slack == 0) return VI_OK;
    VI_REQUIRE(seed_dev && out, "row_prg: null pointer");
    int64_t total = n_rows * slack;
    const int block = 256;
    int64_t grid = (total + block - 1) / block;
    if (grid > 0x7FFFFFFFLL) return vi::fail(VI_ERR_LIMIT, "row_prg: too many elements");
    vi::ProfScope prof(vi::PROF_PRG, (cudaStream_t)stream);
    k_row_prg<<<(unsigned)grid, block, 0, (cudaStream_t)stream>>>(seed_dev, row_off, rows_dev, n_rows, slack, out);
    return vi::check_launch("k_row_prg");
}

extern "C" int vi_challenge(const uint8_t* seed_dev, const uint8_t* label_dev, int label_len,
                            const uint64_t* cids_dev, int64_t n, uint64_t* out, void* stream) {
    VI_REQUIRE(n >= 0, "challenge: negative size");
    VI_REQUIRE(label_len >= 0 && label_len <= 8, "challenge: label must be <= 8 bytes");
    if (n == 0) return VI_OK;
    VI_REQUIRE(seed_dev && out && (label_len == 0 || label_dev), "challenge: null pointer");
    const int block = 256;
    int64_t grid = (n + block - 1) / block;
    if (grid > 0x7FFFFFFFLL) return vi::fail(VI_ERR_LIMIT, "challenge: too many elements");
    k_challenge<<<(unsigned)grid, block, 0, (cudaStream_t)stream>>>(seed_dev, label_dev, label_len, cids_dev, n, out);
    return vi::check_launch("k_challenge");
}

// ---------------------------------------------------------------------------
// Column hash for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the moment they need a column
// hash: a prover that has already handed every free byte of HBM to its witness and
// codeword buffers (an allocation would fail or force it to shrink a buffer), code
// running under a fixed memory budget that forbids driver allocations after start-up,
// or a latency-critical loop in which an allocation's implicit device synchronisation
// is not acceptable.  For them the chaining-value state that vi_hash_columns takes as
// caller scratch lives in the fixed device array below instead.
//
// The array belongs to the library image: every GPU that loads the library holds its
// 8 MiB until the process exits.  All calls (on one device) share it and it keeps the
// contents of the last call.  Nothing in it has to start at zero - each level of the
// state is written before it is read within a call - but two calls that overlap on the
// GPU (different streams, or different host threads) race on it and must be serialised
// by the caller.
//
// The array's device address is looked up on the first call on each device and kept for the life
// of the process: a cudaDeviceReset() on that device invalidates it, so a host that resets a device
// must not call this entry point on it afterwards.  Every input takes the one-thread-per-column
// path; vi_hash_columns cuts matrices with fewer than 131072 columns into concurrent row segments
// (which needs more scratch than this array holds), so narrow inputs get the same digests here but
// take longer than through vi_hash_columns.
// ---------------------------------------------------------------------------
namespace {
constexpr int64_t NOALLOC_STATE_BYTES = int64_t(8) << 20;
static __device__ __align__(256) unsigned char g_noalloc_state[NOALLOC_STATE_BYTES];
constexpr int MAX_DEVICES = 64;
std::mutex g_noalloc_mu;
void* g_noalloc_ptr[MAX_DEVICES] = {};
}  // namespace

extern "C" int64_t vi_hash_columns_noalloc_max_state_bytes(void) { return NOALLOC_STATE_BYTES; }

extern "C" int vi_hash_columns_noalloc(const uint64_t* mat, int64_t m, int64_t ncols, uint8_t* digests,
                                       void* stream) {
    VI_REQUIRE(m >= 0 && ncols >= 0, "hash_columns_noalloc: negative size");
    if (ncols == 0) return VI_OK;
    const int64_t need = m > CHUNK_ROWS ? vi_hash_stream_state_bytes(ncols, m) : 0;
    if (need > NOALLOC_STATE_BYTES)
        return vi::fail(VI_ERR_LIMIT,
                        "hash_columns_noalloc: %lld rows x %lld columns need %lld bytes of chaining-value state, "
                        "the built-in buffer holds %lld; use vi_hash_columns with caller scratch",
                        (long long)m, (long long)ncols, (long long)need, (long long)NOALLOC_STATE_BYTES);
    int dev = 0;
    VI_CUDA(cudaGetDevice(&dev));
    VI_REQUIRE(dev >= 0 && dev < MAX_DEVICES, "hash_columns_noalloc: device index %d not supported", dev);
    void* state = nullptr;
    {
        // Set-up, once per device, with that device current: in host code the array's name is only a
        // stand-in for the symbol, so its device address has to be asked for.
        std::lock_guard<std::mutex> lk(g_noalloc_mu);
        if (!g_noalloc_ptr[dev]) {
            void* p = nullptr;
            VI_CUDA(cudaGetSymbolAddress(&p, g_noalloc_state));
            g_noalloc_ptr[dev] = p;
        }
        state = g_noalloc_ptr[dev];
    }
    return vi_hash_stream_update(state, ncols, m, 0, mat, m, digests, stream);
}
