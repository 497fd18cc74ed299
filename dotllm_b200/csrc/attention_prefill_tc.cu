// Prefill attention on the fifth-generation tensor cores: packed new tokens of several sequences
// over their paged bfloat16 cache, causal, optional sliding window.
//
// Role of the reference's attention_f16 with seq_q > 1 (native/kernels/attention.cu:19-197): scores
// scaled by 1/sqrt(hd), softmax with the running maximum subtracted, weighted sum of values, query
// head h reading KV head h / group.
//
// One block per (tile of 128 query rows, query head).  The cache's layouts are the tensor core's
// K-major operands as they lie: a K page [64 keys][hd] is B of S = Q K^T, a transposed V page
// [hd][64 keys] is B of O += P V.  Six warps with fixed roles:
//   warp 0     tensor-map copies (TMA, 128-byte swizzle): the Q tile once, then K and V pages through
//              a ring of four stages;
//   warp 1     one thread issues tcgen05.mma: S(j) = Q K_j^T into one of two 64-column score buffers
//              in tensor memory, and O += P(j-1) V(j-1) behind it, so that the tensor core computes the
//              next page's scores while the softmax warps work on this page's;
//   warps 2-5  softmax, one query row per thread (tensor-memory lane = row): read the row's 64
//              scores with tcgen05.ld, mask, running maximum and sum in float32 (base 2), write
//              P as bfloat16 into shared memory in the operand's swizzled layout.  O stays in tensor
//              memory for the whole tile; it is rescaled only when a row's maximum has grown by more
//              than 2^8 since the last rescale (the weights stay below 2^8 meanwhile, which bfloat16
//              and the float32 sums hold without loss), and divided by the row's sum at the end.
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

#define PT_ROWS 128
#define PT_STAGES 4
#define PT_THREADS 192
#define PT_TMEM_COLS 256
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
// clock64 at ten points of every page into pt_timeline, which dl_attention_prefill_tc_timeline
// copies out: a per-page timeline of the issuing thread and of one softmax warp
// (`python -m dotllm_b200.kernels.microbench attention_prefill --timeline` prints it).
#ifdef PT_TIMELINE
#define PT_TIMELINE_PAGES 256
__device__ long long pt_timeline[10][PT_TIMELINE_PAGES];
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

template <int HD>
__global__ void __launch_bounds__(PT_THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                            const __grid_constant__ CUtensorMap tmap_v, __nv_bfloat16* __restrict__ out, int out_stride,
                            int n_pages, const int32_t* __restrict__ tile_seq, const int32_t* __restrict__ tile_row0,
                            const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_new,
                            const int32_t* __restrict__ cu_new, const int32_t* __restrict__ block_table, int bt_stride,
                            int nkv, int group, float scale, int window, int* __restrict__ status) {
    constexpr int ATOMS = HD / 64;                           // 64-dim (128-byte) slices of a head
    constexpr uint32_t Q_BYTES = PT_ROWS * HD * 2;
    constexpr uint32_t K_BYTES = DL_PAGE * HD * 2, V_BYTES = HD * DL_PAGE * 2;
    constexpr uint32_t STAGE_BYTES = K_BYTES + V_BYTES;
    constexpr uint32_t P_BYTES = PT_ROWS * DL_PAGE * 2;
    extern __shared__ unsigned char pt_smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)pt_smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_smem = base;                            // [atom][128 rows][64 dims]
    unsigned char* kv_smem = q_smem + Q_BYTES;               // [stage][K: [atom][64 keys][64 dims] | V: [hd][64 keys]]
    unsigned char* p_smem = kv_smem + PT_STAGES * STAGE_BYTES;   // [2][128 rows][64 keys]
    __shared__ uint64_t q_full, kv_full[PT_STAGES], kv_empty[PT_STAGES], s_full[2], s_empty[2], p_ready[2], pv_done[2];
    __shared__ uint32_t tmem_base_holder;
    __shared__ volatile int gave_up;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = gridDim.x - 1 - blockIdx.x;             // later tiles see more keys: start them first
    const int head = blockIdx.y, kvh = head / group;
    const int b = tile_seq[tile], row0 = tile_row0[tile];
    const int start = seq_start[b], n_new = seq_new[b];
    const int rows = min(PT_ROWS, n_new - row0);             // live rows of the tile
    const int pos0 = start + row0;                           // position of the tile's first row
    const int pos_last = pos0 + rows - 1;
    const int total = start + n_new;                         // keys the sequence holds after this step
    const int first_key = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int page_lo = first_key / DL_PAGE, page_hi = pos_last / DL_PAGE;
    const int n_kv = page_hi - page_lo + 1;                  // pages this tile walks

    if (threadIdx.x == 0) {
        gave_up = 0;
        tc_mbar_init(&q_full, 1);
        for (int s = 0; s < PT_STAGES; ++s) {
            tc_mbar_init(&kv_full[s], 1);
            tc_mbar_init(&kv_empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            tc_mbar_init(&s_full[i], 1);
            tc_mbar_init(&s_empty[i], 4);                     // one arrival per softmax warp
            tc_mbar_init(&p_ready[i], 4);
            tc_mbar_init(&pv_done[i], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tc_tmem_alloc(&tmem_base_holder, PT_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_holder;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;    // S0 at 0, S1 at 64, O at 128 ..

    if (warp == 0) {
        // ------------------------------------------------------------ copies
        bool stop = false;
        int issued = 0;
        if (lane == 0) {
            tc_mbar_expect(&q_full, Q_BYTES);
#pragma unroll
            for (int a = 0; a < ATOMS; ++a)
                dl_tma_load_2d(q_smem + a * (PT_ROWS * 128), &tmap_q, head * HD + a * 64, cu_new[b] + row0, &q_full);
        }
        const int32_t* pages = block_table + (size_t)b * bt_stride + page_lo;
        for (int j0 = 0; j0 < n_kv && !stop; j0 += 32) {
            const int mine = (j0 + lane < n_kv) ? pages[j0 + lane] : 0;
            const int count = min(32, n_kv - j0);
            for (int jj = 0; jj < count; ++jj) {
                const int page = __shfl_sync(0xffffffffu, mine, jj);
                const int j = j0 + jj, s = j % PT_STAGES;
                int bad = 0;
                if (lane == 0) {
                    if (page < 0 || page >= n_pages) {
                        bad = 2;
                    } else if (j >= PT_STAGES && !tc_mbar_wait(&kv_empty[s], ((j / PT_STAGES) - 1) & 1, &gave_up)) {
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
            long long t0 = clock64();
            while (!tc_mbar_try(&q_full, 0) && clock64() - t0 < TC_WAIT_CYCLES) {}
            for (int i = max(0, issued - PT_STAGES); i < issued; ++i) {
                t0 = clock64();
                while (!tc_mbar_try(&kv_full[i % PT_STAGES], (i / PT_STAGES) & 1) && clock64() - t0 < TC_WAIT_CYCLES) {}
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ tensor-core issue
        if (lane == 0) {
            const uint32_t idesc_qk = tc_idesc_bf16(PT_ROWS, DL_PAGE), idesc_pv = tc_idesc_bf16(PT_ROWS, HD);
            const uint32_t q_addr = tc_smem(q_smem), p_addr = tc_smem(p_smem);
            bool ok = tc_mbar_wait(&q_full, 0, &gave_up);
            if (!ok && !gave_up) atomicExch(status, 32);
            // page j's product with V is issued behind page j+1's scores
            for (int j = 0; j <= n_kv && ok; ++j) {
                if (j < n_kv) {
                    const int s = j % PT_STAGES, sb = j & 1;
                    PT_STAMP(0, j);                             // issuing thread: top of page j
                    ok = tc_mbar_wait(&kv_full[s], (j / PT_STAGES) & 1, &gave_up) &&
                         (j < 2 || tc_mbar_wait(&s_empty[sb], ((j >> 1) - 1) & 1, &gave_up));
                    if (!ok) {
                        if (!gave_up) atomicExch(status, 33);
                        break;
                    }
                    tc_fence_after();
                    const uint32_t k_addr = tc_smem(kv_smem + (size_t)s * STAGE_BYTES);
#pragma unroll
                    for (int k = 0; k < HD / 16; ++k) {
                        const int a = k / 4, kk = k % 4;        // 64-dim slice, 16-dim step inside it (32 bytes)
                        tc_mma(tmem_s + (uint32_t)(sb * DL_PAGE), tc_operand_desc(q_addr + a * (PT_ROWS * 128)) + (uint64_t)(kk * 2),
                               tc_operand_desc(k_addr + a * (DL_PAGE * 128)) + (uint64_t)(kk * 2), idesc_qk, k != 0 ? 1u : 0u);
                    }
                    tc_commit(&s_full[sb]);
                    PT_STAMP(1, j);                             // scores of page j issued and committed
                }
                if (j >= 1) {
                    const int i = j - 1, s = i % PT_STAGES, pb = i & 1;
                    PT_STAMP(2, i);                             // waiting for the weights of page i
                    ok = tc_mbar_wait(&p_ready[pb], (i >> 1) & 1, &gave_up);
                    PT_STAMP(3, i);                             // weights of page i seen
                    if (!ok) {
                        if (!gave_up) atomicExch(status, 34);
                        break;
                    }
                    tc_fence_after();
                    const uint32_t v_addr = tc_smem(kv_smem + (size_t)s * STAGE_BYTES + K_BYTES);
#pragma unroll
                    for (int k = 0; k < DL_PAGE / 16; ++k)
                        tc_mma(tmem_o, tc_operand_desc(p_addr + pb * P_BYTES) + (uint64_t)(k * 2), tc_operand_desc(v_addr) + (uint64_t)(k * 2),
                               idesc_pv, (i | k) != 0 ? 1u : 0u);
                    tc_commit(&kv_empty[s]);
                    tc_commit(&pv_done[pb]);
                    PT_STAMP(4, i);                             // product of page i issued and committed
                }
            }
            if (!ok) gave_up = 1;
        }
    } else {
        // ------------------------------------------------------------ softmax: thread -> row
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;                   // row of the tile = lane of tensor memory
        const int pos = pos0 + r;
        const bool live = r < rows;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const float scale2 = scale * 1.4426950408889634f;    // scores in units of log2
        float m_ref = -INFINITY, l = 0.f;                    // reference maximum (log2 units), sum of weights
        bool ok = true;
        for (int j = 0; j < n_kv; ++j) {
            const int sb = j & 1;
            if (warp == 2 && lane == 0) PT_STAMP(5, j);         // softmax warp: waiting for the scores of page j
            ok = __all_sync(0xffffffffu, tc_mbar_wait(&s_full[sb], (j >> 1) & 1, &gave_up));
            if (warp == 2 && lane == 0) PT_STAMP(6, j);         // scores seen
            if (!ok) {
                if (lane == 0 && !gave_up) atomicExch(status, 35);
                break;
            }
            tc_fence_after();
            float sc[64];
            {
                float half[32];
                tc_tmem_load32(tmem_s + lane_base + (uint32_t)(sb * DL_PAGE), half);
#pragma unroll
                for (int i = 0; i < 32; ++i) sc[i] = half[i];
                tc_tmem_load32(tmem_s + lane_base + (uint32_t)(sb * DL_PAGE + 32), half);
#pragma unroll
                for (int i = 0; i < 32; ++i) sc[32 + i] = half[i];
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(&s_empty[sb]);        // the score buffer may take page j + 2
            if (warp == 2 && lane == 0) PT_STAMP(7, j);         // scores read into registers

            const int key0 = (page_lo + j) * DL_PAGE;
            // pages wholly visible to every row of the tile need no mask
            const bool ragged = rows < PT_ROWS || key0 + DL_PAGE - 1 > pos0 || key0 < first_key ||
                                (window > 0 && key0 <= pos_last - window);
            if (ragged) {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const int key = key0 + i;
                    const bool seen = live && key <= pos && (window == 0 || key > pos - window);
                    if (!seen) sc[i] = -INFINITY;
                }
            }
            float mx = sc[0];
#pragma unroll
            for (int i = 1; i < 64; ++i) mx = fmaxf(mx, sc[i]);
            mx *= scale2;                                    // scale > 0: the maximum of the scaled scores
            const bool grow = mx > m_ref + PT_RESCALE_STEP || (m_ref == -INFINITY && mx > -INFINITY);
            const bool rescale = __any_sync(0xffffffffu, grow);   // the warp decides: tensor-memory accesses are warp-wide
            float corr = 1.f;
            if (rescale) {
                const float m_new = fmaxf(m_ref, mx);
                corr = (m_new == -INFINITY) ? 1.f : pt_ex2(m_ref - m_new);
                m_ref = m_new;
                l *= corr;
            }
            // the P buffer is free once the product of page j - 2 has finished
            if (warp == 2 && lane == 0) PT_STAMP(8, j);         // maximum done
            if (j >= 2) ok = tc_mbar_wait(&pv_done[sb], ((j >> 1) - 1) & 1, &gave_up);
            // rescaling O needs the product of page j - 1 finished too (it is the other buffer's barrier)
            if (ok && rescale && j >= 1) ok = tc_mbar_wait(&pv_done[sb ^ 1], ((j - 1) >> 1) & 1, &gave_up);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0 && !gave_up) atomicExch(status, 36);
                break;
            }
            if (rescale && j >= 1) {
                tc_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    float o[32];
                    tc_tmem_load32(tmem_o + lane_base + (uint32_t)c0, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] *= corr;
                    tc_tmem_store32(tmem_o + lane_base + (uint32_t)c0, o);
                }
                tc_fence_before();
            }
            // weights of this page, as the A operand of P V: row r is 128 bytes, its 16-byte chunk c at c ^ (r & 7)
            const float sub = (m_ref == -INFINITY) ? 0.f : m_ref;
            const uint32_t p_row = tc_smem(p_smem + sb * P_BYTES) + (uint32_t)r * 128u;
            float sum = 0.f;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                float p[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    p[i] = pt_ex2(fmaf(sc[8 * c + i], scale2, -sub));
                    sum += p[i];
                }
                pt_sts128(p_row + (uint32_t)((c ^ (r & 7)) << 4), pt_pack(p[0], p[1]), pt_pack(p[2], p[3]), pt_pack(p[4], p[5]),
                          pt_pack(p[6], p[7]));
            }
            l += sum;
            // Slots of the sequence's last page beyond its length may hold anything: make them exact
            // zeros in the V stage (row d of V^T is 128 bytes, key k in chunk (k / 8) ^ (d & 7)).
            if (key0 + DL_PAGE > total) {
                unsigned char* v_stage = kv_smem + (size_t)(j % PT_STAGES) * STAGE_BYTES + K_BYTES;
                const int kz = total - key0;                 // first dead key of the page (> 0: the page holds live keys)
                for (int d = r; d < HD; d += PT_ROWS)
                    for (int k = kz; k < DL_PAGE; ++k)
                        *reinterpret_cast<__nv_bfloat16*>(v_stage + d * 128 + ((((k >> 3) ^ (d & 7)) << 4) | ((k & 7) << 1))) =
                            __float2bfloat16_rn(0.f);
            }
            tc_fence_async_smem();                           // shared-memory writes -> the tensor core's reads
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(&p_ready[sb]);
            if (warp == 2 && lane == 0) PT_STAMP(9, j);         // weights stored and announced
        }
        // ---- O / l -> out
        if (ok && n_kv > 0) {
            const int last = n_kv - 1;
            ok = __all_sync(0xffffffffu, tc_mbar_wait(&pv_done[last & 1], (last >> 1) & 1, &gave_up));
            if (!ok && lane == 0 && !gave_up) atomicExch(status, 37);
        }
        if (!ok) gave_up = 1;
        if (ok) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* dst = out + (size_t)(cu_new[b] + row0 + r) * out_stride + (size_t)head * HD;
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 32) {
                float o[32];
                tc_tmem_load32(tmem_o + lane_base + (uint32_t)c0, o);
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
    const size_t smem = (size_t)PT_ROWS * HD * 2 + (size_t)PT_STAGES * 2 * DL_PAGE * HD * 2 + 2 * PT_ROWS * DL_PAGE * 2 + 1024;
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
// 128-row tile its sequence and its first row among that sequence's new tokens.  seq_start,
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
    DL_REQUIRE(nh <= 65535 && (long long)n_pages * nkv * (hd > DL_PAGE ? hd : DL_PAGE) < (1ll << 31),
               "attention_prefill_tc: too many heads or pages");
    if (n_tiles == 0) return DL_OK;
    dim3 grid(n_tiles, nh);
    cudaStream_t s = (cudaStream_t)stream;
    if (hd == 64)
        return pt_launch<64>(grid, s, q, q_stride, n_tokens, out, out_stride, k_pool, v_pool, n_pages, tile_seq, tile_row0,
                             seq_start, seq_new, cu_new, block_table, bt_stride, nh, nkv, scale, window, status);
    if (hd == 128)
        return pt_launch<128>(grid, s, q, q_stride, n_tokens, out, out_stride, k_pool, v_pool, n_pages, tile_seq, tile_row0,
                              seq_start, seq_new, cu_new, block_table, bt_stride, nh, nkv, scale, window, status);
    return dl_fail(DL_ERR_UNSUPPORTED, "attention_prefill_tc: head_dim %d (takes 64 and 128)", hd);
}
