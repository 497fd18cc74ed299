// Prefill attention on the fifth-generation tensor cores: packed new tokens of several sequences
// over their paged bfloat16 cache, causal, optional sliding window.
//
// Role of the reference's attention_f16 with seq_q > 1 (native/kernels/attention.cu:19-197): scores
// scaled by 1/sqrt(hd), softmax with the running maximum subtracted, weighted sum of values, query
// head h reading KV head h / group.
//
// One block per (256 consecutive query rows of a sequence, query head): two tiles of 128 rows that
// share the K and V pages they walk.  The cache's layouts are the tensor core's K-major operands as
// they lie: a K page [64 keys][hd] is B of S = Q K^T, a transposed V page [hd][64 keys] is B of
// O += P V.  Twelve warps with fixed roles:
//   warp 0       tensor-map copies (TMA, 128-byte swizzle): the two Q tiles once, then K and V pages
//                through a ring of stages;
//   warps 1, 2   one thread each issues the tcgen05.mma of one tile's scores: S(j) = Q K_j^T into one
//                of the tile's two 64-column score buffers in tensor memory, so that the tensor core
//                computes the next page's scores while the softmax warps work on this page's;
//   warp 3       one thread issues both tiles' O += P(j) V(j) as their weights become ready, and hands
//                the stage back when every tile that reads the page has had its product issued;
//   warps 4-7    softmax of tile 0, warps 8-11 of tile 1, one query row per thread (tensor-memory lane
//                = row): read the row's 64 scores with tcgen05.ld, mask, running maximum and sum in
//                float32 (base 2), write P as bfloat16 into shared memory in the operand's swizzled
//                layout.  O stays in tensor memory for the whole tile; it is rescaled only when a
//                row's maximum has grown by more than 2^8 since the last rescale (the weights stay
//                below 2^8 meanwhile, which bfloat16 and the float32 sums hold without loss), and
//                divided by the row's sum at the end.
// The tensor core takes about as long for an MMA of 64 or 128 columns as for one of 256 (measured),
// so the kernel is bound by the number of MMAs: two tiles keep that pipe fed while each tile's
// softmax threads work through their page.  Tensor memory: 4 x 64 columns of scores, 2 x 128 of
// outputs - all 512, which one block per SM (its shared memory) makes safe.
// Keys that no query of the tile may see are never used: masked scores are replaced, not
// multiplied, and the slots of the last page beyond the sequence's length (which may hold
// anything) are zeroed in the V stage before the product.
//
// Every wait on an mbarrier is bounded; on expiry the kernel records a code in `status`, stops
// issuing work, waits (bounded) for copies in flight, frees its tensor memory and returns.
#include "common.cuh"
#include "tma.cuh"
#include "tcgen05.cuh"
#include <mutex>
#include <unordered_map>

#define PT_ROWS 128                          // query rows of a tile
#define PT_TILES 2                           // tiles of a block: it covers PT_TILES * PT_ROWS consecutive rows
#define PT_STAGES(hd) ((hd) > 64 ? 3 : 4)    // K/V pages in flight: what 227 KB of shared memory leave room for
#define PT_THREADS 384
#define PT_TMEM_COLS 512
#define PT_RESCALE_STEP 8.0f                 // log2 units a row's maximum may grow before O is rescaled

__device__ __forceinline__ float pt_ex2(float x) {             // 2^x, 2 ulp; ex2(-inf) = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pt_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void pt_sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// Built with -DPT_TIMELINE (DOTLLM_NVCC_EXTRA), block (0, 0) - the tile with the most pages - stamps
// clock64 at twelve points of every page into pt_timeline, which dl_attention_prefill_tc_timeline
// copies out: a per-page timeline of the issuing thread and of one softmax warp
// (`python -m dotllm_b200.kernels.microbench attention_prefill --timeline` prints it).
#ifdef PT_TIMELINE
#define PT_TIMELINE_PAGES 256
__device__ long long pt_timeline[12][PT_TIMELINE_PAGES];
#define PT_STAMP(row, j)                                                                          \
    do {                                                                                          \
        if (blockIdx.x == 0 && blockIdx.y == 0 && (j) < PT_TIMELINE_PAGES) pt_timeline[row][j] = clock64(); \
    } while (0)
extern "C" int dl_attention_prefill_tc_timeline(long long* out) {
    return cudaMemcpyFromSymbol(out, pt_timeline, sizeof(pt_timeline)) == cudaSuccess ? DL_OK : DL_ERR_LAUNCH;
}
#else
#define PT_STAMP(row, j)
#endif

// Where tile `t` of a block stands: its rows, the keys they may see, and its place in the block's walk.
struct PtTile {
    int rows;                // live rows (0: the tile does not exist)
    int pos0, pos_last;      // positions of its first and last live row
    int first_key;           // first key any of its rows may see
    int j_lo, j_hi;          // the pages of the block's walk it takes part in (j_lo > j_hi: none)
};

template <int HD>
__global__ void __launch_bounds__(PT_THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                            const __grid_constant__ CUtensorMap tmap_v, __nv_bfloat16* __restrict__ out, int out_stride,
                            int n_pages, const int32_t* __restrict__ tile_seq, const int32_t* __restrict__ tile_row0,
                            const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_new,
                            const int32_t* __restrict__ cu_new, const int32_t* __restrict__ block_table, int bt_stride,
                            int nkv, int group, float scale, int window, int* __restrict__ status) {
    constexpr int ATOMS = HD / 64;                           // 64-dim (128-byte) slices of a head
    constexpr int STAGES = PT_STAGES(HD);
    constexpr uint32_t Q_BYTES = PT_ROWS * HD * 2;
    constexpr uint32_t K_BYTES = DL_PAGE * HD * 2, V_BYTES = HD * DL_PAGE * 2;
    constexpr uint32_t STAGE_BYTES = K_BYTES + V_BYTES;
    constexpr uint32_t P_BYTES = PT_ROWS * DL_PAGE * 2;
    extern __shared__ unsigned char pt_smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)pt_smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_smem = base;                            // [tile][atom][128 rows][64 dims]
    unsigned char* kv_smem = q_smem + PT_TILES * Q_BYTES;    // [stage][K: [atom][64 keys][64 dims] | V: [hd][64 keys]]
    unsigned char* p_smem = kv_smem + STAGES * STAGE_BYTES;  // [tile][2][128 rows][64 keys]
    __shared__ uint64_t q_full[PT_TILES], kv_full[STAGES], kv_empty[STAGES];
    __shared__ uint64_t s_full[PT_TILES][2], s_empty[PT_TILES][2], p_ready[PT_TILES][2], pv_done[PT_TILES][2];
    __shared__ uint32_t tmem_base_holder;
    __shared__ volatile int gave_up;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Blocks are handed out with x fastest: all heads of the first tile, then of the second.  The caller
    // lists the tiles with the most keys first, so the long blocks start first and the short ones fill
    // the multiprocessors' last gaps; the heads of a KV group run side by side and share its pages in L2.
    const int blk = blockIdx.y;
    const int head = blockIdx.x, kvh = head / group;
    const int b = tile_seq[blk], row0 = tile_row0[blk];
    const int start = seq_start[b], n_new = seq_new[b];
    const int total = start + n_new;                         // keys the sequence holds after this step
    PtTile tiles[PT_TILES];
#pragma unroll
    for (int t = 0; t < PT_TILES; ++t) {
        PtTile& T = tiles[t];
        T.rows = max(0, min(PT_ROWS, n_new - row0 - t * PT_ROWS));
        T.pos0 = start + row0 + t * PT_ROWS;
        T.pos_last = T.pos0 + T.rows - 1;
        T.first_key = (window > 0 && T.pos0 - window + 1 > 0) ? T.pos0 - window + 1 : 0;
    }
    // The block walks the pages from the first one tile 0 sees to the last one its last live tile sees;
    // a tile joins at its own first page and leaves after its own last (the ranges overlap or touch).
    const int page_lo = tiles[0].first_key / DL_PAGE;
    int page_hi = tiles[0].pos_last / DL_PAGE;
#pragma unroll
    for (int t = 0; t < PT_TILES; ++t) {
        PtTile& T = tiles[t];
        T.j_lo = T.first_key / DL_PAGE - page_lo;
        T.j_hi = T.rows > 0 ? T.pos_last / DL_PAGE - page_lo : T.j_lo - 1;
        if (T.rows > 0) page_hi = max(page_hi, T.pos_last / DL_PAGE);
    }
    const int n_kv = page_hi - page_lo + 1;                  // pages this block walks

    if (threadIdx.x == 0) {
        gave_up = 0;
        for (int s = 0; s < STAGES; ++s) {
            tc_mbar_init(&kv_full[s], 1);
            tc_mbar_init(&kv_empty[s], 1);
        }
        for (int t = 0; t < PT_TILES; ++t) {
            tc_mbar_init(&q_full[t], 1);
            for (int i = 0; i < 2; ++i) {
                tc_mbar_init(&s_full[t][i], 1);
                tc_mbar_init(&s_empty[t][i], 4);              // one arrival per softmax warp of the tile
                tc_mbar_init(&p_ready[t][i], 4);
                tc_mbar_init(&pv_done[t][i], 1);
            }
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tc_tmem_alloc(&tmem_base_holder, PT_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_holder;
    // scores: tile t, buffer i at column (2 t + i) * 64; outputs: tile t at column 256 + 128 t
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 2 * PT_TILES * DL_PAGE;

    if (warp == 0) {
        // ------------------------------------------------------------ copies
        bool stop = false;
        int issued = 0;
        if (lane == 0) {
#pragma unroll
            for (int t = 0; t < PT_TILES; ++t) {
                if (tiles[t].rows <= 0) continue;
                tc_mbar_expect(&q_full[t], Q_BYTES);
#pragma unroll
                for (int a = 0; a < ATOMS; ++a)
                    dl_tma_load_2d(q_smem + t * Q_BYTES + a * (PT_ROWS * 128), &tmap_q, head * HD + a * 64,
                                   cu_new[b] + row0 + t * PT_ROWS, &q_full[t]);
            }
        }
        const int32_t* pages = block_table + (size_t)b * bt_stride + page_lo;
        for (int j0 = 0; j0 < n_kv && !stop; j0 += 32) {
            const int mine = (j0 + lane < n_kv) ? pages[j0 + lane] : 0;
            const int count = min(32, n_kv - j0);
            for (int jj = 0; jj < count; ++jj) {
                const int page = __shfl_sync(0xffffffffu, mine, jj);
                const int j = j0 + jj, s = j % STAGES;
                int bad = 0;
                if (lane == 0) {
                    if (page < 0 || page >= n_pages) {
                        bad = 2;
                    } else if (j >= STAGES && !tc_mbar_wait(&kv_empty[s], ((j / STAGES) - 1) & 1, &gave_up)) {
                        bad = 31;
                    } else {
                        unsigned char* k_dst = kv_smem + (size_t)s * STAGE_BYTES;
                        tc_mbar_expect(&kv_full[s], STAGE_BYTES);
#pragma unroll
                        for (int a = 0; a < ATOMS; ++a)
                            dl_tma_load_2d(k_dst + a * (DL_PAGE * 128), &tmap_k, a * 64, (page * nkv + kvh) * DL_PAGE, &kv_full[s]);
                        dl_tma_load_2d(k_dst + K_BYTES, &tmap_v, 0, (page * nkv + kvh) * HD, &kv_full[s]);
                        issued = j + 1;
                    }
                }
                bad = __shfl_sync(0xffffffffu, bad, 0);
                if (bad) {
                    if (lane == 0) {
                        if (!gave_up) atomicExch(status, bad);
                        gave_up = 1;
                    }
                    stop = true;
                    break;
                }
            }
        }
        if (stop && lane == 0) {
            // copies already issued must land before the block's shared memory is released
            for (int t = 0; t < PT_TILES; ++t) {
                if (tiles[t].rows <= 0) continue;
                const long long t0 = clock64();
                while (!tc_mbar_try(&q_full[t], 0) && clock64() - t0 < TC_WAIT_CYCLES) {}
            }
            for (int i = max(0, issued - STAGES); i < issued; ++i) {
                const long long t0 = clock64();
                while (!tc_mbar_try(&kv_full[i % STAGES], (i / STAGES) & 1) && clock64() - t0 < TC_WAIT_CYCLES) {}
            }
        }
    } else if (warp == 1 || warp == 2) {
        // ------------------------------------------------------------ tensor-core issue: the scores of tile `t`
        const int t = warp - 1;
        const PtTile T = tiles[t];
        if (lane == 0 && T.rows > 0) {
            const uint32_t idesc_qk = tc_idesc_bf16(PT_ROWS, DL_PAGE);
            const uint32_t q_addr = tc_smem(q_smem + t * Q_BYTES);
            bool ok = tc_mbar_wait(&q_full[t], 0, &gave_up);
            if (!ok && !gave_up) atomicExch(status, 32);
            for (int j = T.j_lo; j <= T.j_hi && ok; ++j) {
                const int c = j - T.j_lo, s = j % STAGES, sb = c & 1;
                if (t == 0) PT_STAMP(0, j);                     // issuing thread: top of page j
                ok = tc_mbar_wait(&kv_full[s], (j / STAGES) & 1, &gave_up) &&
                     (c < 2 || tc_mbar_wait(&s_empty[t][sb], ((c >> 1) - 1) & 1, &gave_up));
                if (!ok) {
                    if (!gave_up) atomicExch(status, 33);
                    break;
                }
                tc_fence_after();
                const uint32_t k_addr = tc_smem(kv_smem + (size_t)s * STAGE_BYTES);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const int a = k / 4, kk = k % 4;            // 64-dim slice, 16-dim step inside it (32 bytes)
                    tc_mma(tmem_s + (uint32_t)((2 * t + sb) * DL_PAGE), tc_operand_desc(q_addr + a * (PT_ROWS * 128)) + (uint64_t)(kk * 2),
                           tc_operand_desc(k_addr + a * (DL_PAGE * 128)) + (uint64_t)(kk * 2), idesc_qk, k != 0 ? 1u : 0u);
                }
                tc_commit(&s_full[t][sb]);
                if (t == 0) PT_STAMP(1, j);                     // scores of page j issued and committed
            }
            if (!ok) gave_up = 1;
        }
    } else if (warp == 3) {
        // ------------------------------------------------------------ tensor-core issue: the products with V
        if (lane == 0) {
            const uint32_t idesc_pv = tc_idesc_bf16(PT_ROWS, HD);
            bool ok = true;
            for (int j = 0; j < n_kv && ok; ++j) {
                const int s = j % STAGES;
                const uint32_t v_addr = tc_smem(kv_smem + (size_t)s * STAGE_BYTES + K_BYTES);
#pragma unroll
                for (int t = 0; t < PT_TILES; ++t) {
                    if (j < tiles[t].j_lo || j > tiles[t].j_hi) continue;
                    const int c = j - tiles[t].j_lo, pb = c & 1;
                    if (t == 0) PT_STAMP(2, j);                 // waiting for the weights of page j
                    ok = tc_mbar_wait(&p_ready[t][pb], (c >> 1) & 1, &gave_up) && tc_mbar_wait(&kv_full[s], (j / STAGES) & 1, &gave_up);
                    if (t == 0) PT_STAMP(3, j);                 // weights of page j seen
                    if (!ok) {
                        if (!gave_up) atomicExch(status, 34);
                        break;
                    }
                    tc_fence_after();
                    const uint32_t p_addr = tc_smem(p_smem + (2 * t + pb) * P_BYTES);
#pragma unroll
                    for (int k = 0; k < DL_PAGE / 16; ++k)
                        tc_mma(tmem_o + (uint32_t)(t * HD), tc_operand_desc(p_addr) + (uint64_t)(k * 2), tc_operand_desc(v_addr) + (uint64_t)(k * 2),
                               idesc_pv, (c | k) != 0 ? 1u : 0u);
                    tc_commit(&pv_done[t][pb]);
                    if (t == 0) PT_STAMP(4, j);                 // product of page j issued and committed
                }
                if (ok) tc_commit(&kv_empty[s]);                // every tile that reads this page has issued its product
            }
            if (!ok) gave_up = 1;
        }
    } else {
        // ------------------------------------------------------------ softmax: thread -> row of tile `t`
        const int t = (warp - 4) >> 2, quarter = warp & 3;
        const PtTile T = tiles[t];
        const int r = quarter * 32 + lane;                   // row of the tile = lane of tensor memory
        const int pos = T.pos0 + r;
        const bool live = r < T.rows;
        const bool stamps = (warp == 4 && lane == 0);
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t my_s = tmem_s + lane_base + (uint32_t)(2 * t * DL_PAGE), my_o = tmem_o + lane_base + (uint32_t)(t * HD);
        const float scale2 = scale * 1.4426950408889634f;    // scores in units of log2
        float m_ref = -INFINITY, l = 0.f;                    // reference maximum (log2 units), sum of weights
        bool ok = true;
        const int n_mine = T.j_hi - T.j_lo + 1;
        for (int c = 0; c < n_mine; ++c) {
            const int j = T.j_lo + c, sb = c & 1;
            if (stamps) PT_STAMP(5, j);                         // softmax warp: waiting for the scores of page j
            ok = __all_sync(0xffffffffu, tc_mbar_wait(&s_full[t][sb], (c >> 1) & 1, &gave_up));
            if (stamps) PT_STAMP(6, j);                         // scores seen
            if (!ok) {
                if (lane == 0 && !gave_up) atomicExch(status, 35);
                break;
            }
            tc_fence_after();
            float sc[64];
            {
                float half[32];
                tc_tmem_load32(my_s + (uint32_t)(sb * DL_PAGE), half);
#pragma unroll
                for (int i = 0; i < 32; ++i) sc[i] = half[i];
                tc_tmem_load32(my_s + (uint32_t)(sb * DL_PAGE + 32), half);
#pragma unroll
                for (int i = 0; i < 32; ++i) sc[32 + i] = half[i];
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(&s_empty[t][sb]);     // the score buffer may take the tile's page after next
            if (stamps) PT_STAMP(7, j);                         // scores read into registers

            const int key0 = (page_lo + j) * DL_PAGE;
            // pages wholly visible to every row of the tile need no mask
            const bool ragged = T.rows < PT_ROWS || key0 + DL_PAGE - 1 > T.pos0 || key0 < T.first_key ||
                                (window > 0 && key0 <= T.pos_last - window);
            if (ragged) {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const int key = key0 + i;
                    const bool seen = live && key <= pos && (window == 0 || key > pos - window);
                    if (!seen) sc[i] = -INFINITY;
                }
            }
            float mx4[4] = {sc[0], sc[1], sc[2], sc[3]};     // four chains: a single one is 64 dependent steps
#pragma unroll
            for (int i = 4; i < 64; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], sc[i]);
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale2;   // scale > 0: the maximum of the scaled scores
            const bool grow = mx > m_ref + PT_RESCALE_STEP || (m_ref == -INFINITY && mx > -INFINITY);
            const bool rescale = __any_sync(0xffffffffu, grow);   // the warp decides: tensor-memory accesses are warp-wide
            float corr = 1.f;
            if (rescale) {
                const float m_new = fmaxf(m_ref, mx);
                corr = (m_new == -INFINITY) ? 1.f : pt_ex2(m_ref - m_new);
                m_ref = m_new;
                l *= corr;
            }
            if (stamps) PT_STAMP(8, j);                         // maximum done
            // the P buffer is free once the product of the tile's page before last has finished
            if (c >= 2) ok = tc_mbar_wait(&pv_done[t][sb], ((c >> 1) - 1) & 1, &gave_up);
            // rescaling O needs the product of the page before finished too (it is the other buffer's barrier)
            if (ok && rescale && c >= 1) ok = tc_mbar_wait(&pv_done[t][sb ^ 1], ((c - 1) >> 1) & 1, &gave_up);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0 && !gave_up) atomicExch(status, 36);
                break;
            }
            if (stamps) PT_STAMP(10, j);                        // the weights' buffer is free
            if (rescale && c >= 1) {
                tc_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    float o[32];
                    tc_tmem_load32(my_o + (uint32_t)c0, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] *= corr;
                    tc_tmem_store32(my_o + (uint32_t)c0, o);
                }
                tc_fence_before();
            }
            // weights of this page, as the A operand of P V: row r is 128 bytes, its 16-byte chunk c at c ^ (r & 7)
            const float sub = (m_ref == -INFINITY) ? 0.f : m_ref;
            const uint32_t p_row = tc_smem(p_smem + (2 * t + sb) * P_BYTES) + (uint32_t)r * 128u;
            // all exponentials first, in place: the special-function unit takes them back to back, and the
            // sums, the packing and the stores follow in its shadow
#pragma unroll
            for (int i = 0; i < 64; ++i) sc[i] = pt_ex2(fmaf(sc[i], scale2, -sub));
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 64; ++i) sum4[i & 3] += sc[i];
            l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
                const float* p = sc + 8 * ch;
                pt_sts128(p_row + (uint32_t)((ch ^ (r & 7)) << 4), pt_pack(p[0], p[1]), pt_pack(p[2], p[3]), pt_pack(p[4], p[5]),
                          pt_pack(p[6], p[7]));
            }
            // Slots of the sequence's last page beyond its length may hold anything: make them exact
            // zeros in the V stage (row d of V^T is 128 bytes, key k in chunk (k / 8) ^ (d & 7)).  Both
            // tiles may do this to the same page; they write the same zeros.
            if (key0 + DL_PAGE > total) {
                unsigned char* v_stage = kv_smem + (size_t)(j % STAGES) * STAGE_BYTES + K_BYTES;
                const int kz = total - key0;                 // first dead key of the page (> 0: the page holds live keys)
                for (int d = r; d < HD; d += PT_ROWS)
                    for (int k = kz; k < DL_PAGE; ++k)
                        *reinterpret_cast<__nv_bfloat16*>(v_stage + d * 128 + ((((k >> 3) ^ (d & 7)) << 4) | ((k & 7) << 1))) =
                            __float2bfloat16_rn(0.f);
            }
            if (stamps) PT_STAMP(11, j);                        // weights stored
            tc_fence_async_smem();                           // shared-memory writes -> the tensor core's reads
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(&p_ready[t][sb]);
            if (stamps) PT_STAMP(9, j);                         // weights stored and announced
        }
        // ---- O / l -> out
        if (ok && n_mine > 0) {
            const int last = n_mine - 1;
            ok = __all_sync(0xffffffffu, tc_mbar_wait(&pv_done[t][last & 1], (last >> 1) & 1, &gave_up));
            if (!ok && lane == 0 && !gave_up) atomicExch(status, 37);
        }
        if (!ok) gave_up = 1;
        if (ok && n_mine > 0) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* dst = out + (size_t)(cu_new[b] + row0 + t * PT_ROWS + r) * out_stride + (size_t)head * HD;
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 32) {
                float o[32];
                tc_tmem_load32(my_o + (uint32_t)c0, o);
                if (live) {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        *reinterpret_cast<uint4*>(dst + c0 + 8 * i) =
                            make_uint4(pt_pack(o[8 * i] * inv, o[8 * i + 1] * inv), pt_pack(o[8 * i + 2] * inv, o[8 * i + 3] * inv),
                                       pt_pack(o[8 * i + 4] * inv, o[8 * i + 5] * inv), pt_pack(o[8 * i + 6] * inv, o[8 * i + 7] * inv));
                }
            }
            tc_fence_before();
        }
    }
    tc_fence_before();
    __syncthreads();                                         // nobody leaves while copies or MMAs may be in flight
    if (warp == 1) {
        tc_fence_after();
        tc_tmem_free(tmem_base, PT_TMEM_COLS);
    }
}

struct PtMapKey {
    const void* base;
    long long rows, cols, pitch;
    int box_rows;
    bool operator==(const PtMapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && pitch == o.pitch && box_rows == o.box_rows;
    }
};
struct PtMapKeyHash {
    size_t operator()(const PtMapKey& k) const {
        return std::hash<const void*>()(k.base) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.cols * 10007u) ^ ((size_t)k.pitch * 31u) ^
               (size_t)k.box_rows;
    }
};

static int pt_tensor_map(CUtensorMap* out, const void* base, long long rows, long long cols, long long pitch_bytes, int box_rows) {
    static std::unordered_map<PtMapKey, CUtensorMap, PtMapKeyHash> maps;
    static std::mutex maps_mutex;
    std::lock_guard<std::mutex> lock(maps_mutex);
    const PtMapKey key{base, rows, cols, pitch_bytes, box_rows};
    auto it = maps.find(key);
    if (it == maps.end()) {
        CUtensorMap fresh;
        if (dl_tmap_encode_2d_bf16(&fresh, base, (uint64_t)rows, (uint64_t)cols, (uint64_t)pitch_bytes, box_rows, 64,
                                   DL_TMAP_SWIZZLE_128B) != 0)
            return DL_ERR_LAUNCH;
        if (maps.size() > 4096) maps.clear();
        it = maps.emplace(key, fresh).first;
    }
    *out = it->second;
    return DL_OK;
}

template <int HD>
static int pt_launch(dim3 grid, cudaStream_t s, const void* q, int q_stride, int n_tokens, void* out, int out_stride,
                     const void* k_pool, const void* v_pool, int n_pages, const int32_t* tile_seq, const int32_t* tile_row0,
                     const int32_t* seq_start, const int32_t* seq_new, const int32_t* cu_new, const int32_t* block_table,
                     int bt_stride, int nh, int nkv, float scale, int window, int* status) {
    const size_t smem = (size_t)PT_TILES * PT_ROWS * HD * 2 + (size_t)PT_STAGES(HD) * 2 * DL_PAGE * HD * 2 +
                        (size_t)PT_TILES * 2 * PT_ROWS * DL_PAGE * 2 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "attention_prefill_tc: shared memory %zu: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    CUtensorMap tmap_q, tmap_k, tmap_v;
    int rc = pt_tensor_map(&tmap_q, q, n_tokens, (long long)nh * HD, (long long)q_stride * 2, PT_ROWS);
    if (rc != DL_OK) return rc;
    rc = pt_tensor_map(&tmap_k, k_pool, (long long)n_pages * nkv * DL_PAGE, HD, (long long)HD * 2, DL_PAGE);
    if (rc != DL_OK) return rc;
    rc = pt_tensor_map(&tmap_v, v_pool, (long long)n_pages * nkv * HD, DL_PAGE, (long long)DL_PAGE * 2, HD);
    if (rc != DL_OK) return rc;
    attention_prefill_tc_kernel<HD><<<grid, PT_THREADS, smem, s>>>(tmap_q, tmap_k, tmap_v, (__nv_bfloat16*)out, out_stride, n_pages,
                                                                  tile_seq, tile_row0, seq_start, seq_new, cu_new, block_table,
                                                                  bt_stride, nkv, nh / nkv, scale, window, status);
    DL_CHECK_LAUNCH("attention_prefill_tc");
    return DL_OK;
}

// q, out: bf16 [n_tokens, nh*hd] packed new tokens of all sequences.  tile_seq / tile_row0: for every
// 256-row tile its sequence and its first row among that sequence's new tokens, best with the tiles
// that see the most keys first.  seq_start,
// seq_new: cached length before the step and new tokens, per sequence; cu_new: packed offsets.
// head_dim 64 or 128.  status: int32, set non-zero if a wait expired.
extern "C" int dl_attention_prefill_tc_bf16(const void* q, int q_stride, int n_tokens, void* out, int out_stride,
                                            const void* k_pool, const void* v_pool, int n_pages, const int32_t* tile_seq,
                                            const int32_t* tile_row0, int n_tiles, const int32_t* seq_start,
                                            const int32_t* seq_new, const int32_t* cu_new, const int32_t* block_table,
                                            int bt_stride, int nh, int nkv, int hd, float scale, int window, int* status,
                                            void* stream) {
    DL_REQUIRE(n_tiles >= 0 && n_tokens >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0, "attention_prefill_tc: bad sizes");
    DL_REQUIRE(scale > 0.f && window >= 0, "attention_prefill_tc: the score scale must be positive, the window not negative");
    DL_REQUIRE(status != nullptr, "attention_prefill_tc: needs a status word");
    DL_REQUIRE(q_stride % 8 == 0 && out_stride % 8 == 0 && ((uintptr_t)q % 16) == 0 && ((uintptr_t)out % 16) == 0 &&
                   ((uintptr_t)k_pool % 16) == 0 && ((uintptr_t)v_pool % 16) == 0,
               "attention_prefill_tc: q, out and the pools must be 16-byte aligned with rows a multiple of 16 bytes");
    DL_REQUIRE(q_stride >= nh * hd && out_stride >= nh * hd, "attention_prefill_tc: row strides shorter than the rows");
    DL_REQUIRE((long long)n_pages * nkv * (hd > DL_PAGE ? hd : DL_PAGE) < (1ll << 31),
               "attention_prefill_tc: too many heads or pages");
    if (n_tiles == 0) return DL_OK;
    DL_REQUIRE(n_tiles <= 65535, "attention_prefill_tc: too many tiles (%d)", n_tiles);
    dim3 grid(nh, n_tiles);
    cudaStream_t s = (cudaStream_t)stream;
    if (hd == 64)
        return pt_launch<64>(grid, s, q, q_stride, n_tokens, out, out_stride, k_pool, v_pool, n_pages, tile_seq, tile_row0,
                             seq_start, seq_new, cu_new, block_table, bt_stride, nh, nkv, scale, window, status);
    if (hd == 128)
        return pt_launch<128>(grid, s, q, q_stride, n_tokens, out, out_stride, k_pool, v_pool, n_pages, tile_seq, tile_row0,
                              seq_start, seq_new, cu_new, block_table, bt_stride, nh, nkv, scale, window, status);
    return dl_fail(DL_ERR_UNSUPPORTED, "attention_prefill_tc: head_dim %d (takes 64 and 128)", hd);
}
