// Prefill attention: many new tokens per sequence (whole prompts or chunks) over the paged
// bfloat16 cache, causal, optionally windowed, packed sequences of unequal lengths.
//
// Role of the reference's attention_f16 with seq_q > 1 (native/kernels/attention.cu:19-197), which
// gives one block to every (query token, head) and walks the keys with scalar dot products.  Here a
// block owns 128 consecutive query positions of one head: eight consumer warps of 16 rows each, the
// rows of mma.sync.m16n8k16 tiles.  One producer thread streams the cache pages the block needs
// (K [64][hd] and V [hd][64] of the head's KV head, two contiguous pieces per page) with
// cp.async.bulk into a ring of shared-memory stages; every consumer warp reads every page from
// there, so a page crosses from L2 once per 128 rows.  Each warp keeps an online softmax in float32
// registers, in base 2 with ex2.approx (2 ulp, far below the bfloat16 rounding of the weights that
// follows), and masks only the pages that touch its diagonal or the window's edge.  Operand
// fragments use the k-permutation of the decode kernel (csrc/attention_decode.cu).  The new tokens'
// own keys and values are already in the cache when this runs, so one loop covers earlier context
// and the causal triangle.
//
// Every consumer warp waits on every phase of every stage's barrier, in order.  Waits are bounded
// (about a second of clock cycles); on expiry the kernel records a code in `status` and returns
// after waiting (bounded) for copies in flight.
#include "common.cuh"

#define AP_CONSUMERS 8
#define AP_ROWS (16 * AP_CONSUMERS)
#define AP_THREADS (32 * (AP_CONSUMERS + 1))
#define AP_STAGES 4
#define AP_WAIT_CYCLES (1ll << 31)

__device__ __forceinline__ void ap_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    // not volatile: independent accumulators must be free to interleave
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ap_ex2(float x) {            // 2^x, 2 ulp; ex2(-inf) = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t ap_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t ap_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ap_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ap_smem(bar)), "r"(count));
}
__device__ __forceinline__ void ap_mbar_expect(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ap_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ap_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ap_smem(bar)) : "memory");
}
__device__ __forceinline__ bool ap_mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(ap_smem(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool ap_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* gave_up) {
    if (ap_mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (!ap_mbar_try(bar, parity)) {
        if (*gave_up || clock64() - t0 > AP_WAIT_CYCLES) return false;
    }
    return true;
}
__device__ __forceinline__ void ap_bulk_copy(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(ap_smem(dst)),
                 "l"(src), "r"(bytes), "r"(ap_smem(bar))
                 : "memory");
}
__device__ __forceinline__ uint4 ap_lds128(uint32_t addr) {  // 16 bytes from a shared-space byte address
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}

template <int HD>
__global__ void __launch_bounds__(AP_THREADS, 1)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                         int out_stride, const __nv_bfloat16* __restrict__ k_pool,
                         const __nv_bfloat16* __restrict__ v_pool, int n_pages,
                         const int32_t* __restrict__ tile_seq, const int32_t* __restrict__ tile_row0,
                         const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_new,
                         const int32_t* __restrict__ cu_new, const int32_t* __restrict__ block_table,
                         int bt_stride, int nh, int nkv, float scale, int window, int* __restrict__ status) {
    constexpr int DC = HD / 32;
    constexpr int DT = HD / 8;
    constexpr int PAGE_ELEMS = DL_PAGE * HD;
    constexpr uint32_t PAGE_BYTES = PAGE_ELEMS * 2;
    extern __shared__ __align__(128) unsigned char ap_smem_raw[];
    __nv_bfloat16* stage_mem = reinterpret_cast<__nv_bfloat16*>(ap_smem_raw);      // [stage][K page | V page]
    __shared__ uint64_t full_bar[AP_STAGES], empty_bar[AP_STAGES];
    __shared__ volatile int gave_up;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int tile = blockIdx.y, h = blockIdx.x;             // x fastest: all heads of the caller's first (longest) tile start first
    const int b = tile_seq[tile];
    const int tile_row = tile_row0[tile];                // first of the block's rows among the sequence's new tokens
    const int n_new = seq_new[b];
    const int start = seq_start[b];
    const int kvh = h / (nh / nkv);
    const int rows_here = min(AP_ROWS, n_new - tile_row);
    const int n_active = (rows_here + 15) / 16;          // consumer warps that own at least one row
    // keys the block needs: from the first key its first row may see to its last row's own position
    const int blk_pos_min = start + tile_row, blk_pos_max = start + tile_row + rows_here - 1;
    const int blk_first = (window > 0 && blk_pos_min - window + 1 > 0) ? blk_pos_min - window + 1 : 0;
    const int page_lo = blk_first / DL_PAGE, page_hi = blk_pos_max / DL_PAGE;
    const int n_blk_pages = page_hi - page_lo + 1;
    const int32_t* pages = block_table + (size_t)b * bt_stride;

    if (threadIdx.x == 0) {
        gave_up = 0;
        for (int s = 0; s < AP_STAGES; ++s) {
            ap_mbar_init(&full_bar[s], 1);
            ap_mbar_init(&empty_bar[s], n_active);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == AP_CONSUMERS) {
        // ------------------------------------------------------------ producer (one thread)
        if (lane == 0) {
            int n = 0;
            for (; n < n_blk_pages; ++n) {
                const int s = n % AP_STAGES;
                const int page = pages[page_lo + n];
                if (page < 0 || page >= n_pages) { gave_up = 1; atomicExch(status, 2); break; }   // host-validated
                if (n >= AP_STAGES && !ap_mbar_wait(&empty_bar[s], ((n / AP_STAGES) - 1) & 1, &gave_up)) {
                    if (!gave_up) atomicExch(status, 1);
                    gave_up = 1;
                    break;
                }
                __nv_bfloat16* dst = stage_mem + (size_t)s * 2 * PAGE_ELEMS;
                ap_mbar_expect(&full_bar[s], 2 * PAGE_BYTES);
                ap_bulk_copy(dst, k_pool + dl_k_offset(page, nkv, kvh, 0, HD), PAGE_BYTES, &full_bar[s]);
                ap_bulk_copy(dst + PAGE_ELEMS, v_pool + dl_v_offset(page, nkv, kvh, 0, HD), PAGE_BYTES, &full_bar[s]);
            }
            if (gave_up) {
                // copies already issued must land before the block's shared memory is released
                for (int i = max(0, n - AP_STAGES); i < n; ++i) {
                    const long long t0 = clock64();
                    while (!ap_mbar_try(&full_bar[i % AP_STAGES], (i / AP_STAGES) & 1) && clock64() - t0 < AP_WAIT_CYCLES) {}
                }
            }
        }
    } else if (warp < n_active) {
        // ------------------------------------------------------------ consumers: 16 rows each
        const int row0 = tile_row + 16 * warp;
        const int tok0 = cu_new[b] + row0;                   // packed token index of the warp's first row
        const bool ok_lo = row0 + g < n_new, ok_hi = row0 + g + 8 < n_new;
        const int pos_lo = ok_lo ? start + row0 + g : -1;    // rows that do not exist see no key
        const int pos_hi = ok_hi ? start + row0 + g + 8 : -1;
        const int warp_pos_min = start + row0, warp_pos_max = start + min(row0 + 15, n_new - 1);
        const int first_lo = (window > 0) ? pos_lo - window + 1 : 0;
        const int first_hi = (window > 0) ? pos_hi - window + 1 : 0;
        const int warp_first = (window > 0 && warp_pos_min - window + 1 > 0) ? warp_pos_min - window + 1 : 0;
        const float scale2 = scale * 1.4426950408889634f;    // scores in units of log2

        uint4 qf_lo[DC], qf_hi[DC];
#pragma unroll
        for (int c = 0; c < DC; ++c) {
            qf_lo[c] = make_uint4(0u, 0u, 0u, 0u);
            qf_hi[c] = make_uint4(0u, 0u, 0u, 0u);
            if (ok_lo) qf_lo[c] = *reinterpret_cast<const uint4*>(q + (size_t)(tok0 + g) * q_stride + (size_t)h * HD + c * 32 + t * 8);
            if (ok_hi) qf_hi[c] = *reinterpret_cast<const uint4*>(q + (size_t)(tok0 + g + 8) * q_stride + (size_t)h * HD + c * 32 + t * 8);
        }
        float o[DT][4];
#pragma unroll
        for (int i = 0; i < DT; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
        float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;   // maxima in units of log2

        for (int n = 0; n < n_blk_pages; ++n) {
            const int s = n % AP_STAGES;
            if (!ap_mbar_wait(&full_bar[s], (n / AP_STAGES) & 1, &gave_up)) {
                if (!gave_up) atomicExch(status, 3);
                gave_up = 1;
                break;
            }
            const int base = (page_lo + n) * DL_PAGE;        // first key of the page
            // pages wholly outside what this warp's rows may see are only released
            if (base <= warp_pos_max && base + DL_PAGE > warp_first) {
                __nv_bfloat16* kp = stage_mem + (size_t)s * 2 * PAGE_ELEMS;
                const uint32_t k_addr = ap_smem(kp) + (uint32_t)((8 * (g >> 1) + (g & 1)) * HD + t * 8) * 2u;
                const uint32_t v_addr = ap_smem(kp + PAGE_ELEMS) + (uint32_t)(g * DL_PAGE + t * 8) * 2u;
                // masks are needed where the page reaches past the warp's first row or before its window
                const bool ragged = (base + DL_PAGE - 1 > warp_pos_min) || (window > 0 && base < warp_pos_max - window + 1);

                float sc[2][4][4];
#pragma unroll
                for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int e = 0; e < 4; ++e) sc[hh][j][e] = 0.f;
#pragma unroll
                for (int c = 0; c < DC; ++c) {
                    uint4 kf[2][4];
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                        for (int j = 0; j < 4; ++j)     // key 32hh + 8(g/2) + 2j + (g&1), dims 32c + 8t ..
                            kf[hh][j] = ap_lds128(k_addr + (uint32_t)(((32 * hh + 2 * j) * HD + c * 32) * 2));
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            ap_mma(sc[hh][j], qf_lo[c].x, qf_hi[c].x, qf_lo[c].y, qf_hi[c].y, kf[hh][j].x, kf[hh][j].y);
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            ap_mma(sc[hh][j], qf_lo[c].z, qf_hi[c].z, qf_lo[c].w, qf_hi[c].w, kf[hh][j].z, kf[hh][j].w);
                }
                if (ragged) {
                    // lane holds keys base + 32hh + 8t + 2j + {0,1} of rows g (lo) and g+8 (hi).  Masked
                    // scores become -inf, hence weight 0; a value under weight 0 must still be finite,
                    // which holds for every key <= the block's last position (all written), and keys
                    // beyond it are masked for every row, so their weights are exactly 0 too - but a
                    // reused page may hold NaN there, so those values are zeroed in the stage below.
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                        for (int j = 0; j < 4; ++j)
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const int key = base + 32 * hh + 8 * t + 2 * j + e;
                                if (key > pos_lo || key < first_lo) sc[hh][j][e] = -INFINITY;
                                if (key > pos_hi || key < first_hi) sc[hh][j][2 + e] = -INFINITY;
                            }
                }
                float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
                for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        mx_lo = fmaxf(mx_lo, fmaxf(sc[hh][j][0], sc[hh][j][1]));
                        mx_hi = fmaxf(mx_hi, fmaxf(sc[hh][j][2], sc[hh][j][3]));
                    }
                mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
                mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
                mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
                mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
                // scale > 0, so the maximum of the scaled scores is the scaled maximum
                const float mn_lo = fmaxf(m_lo, mx_lo * scale2), mn_hi = fmaxf(m_hi, mx_hi * scale2);
                const bool dead_lo = mn_lo == -INFINITY, dead_hi = mn_hi == -INFINITY;   // nothing seen yet
                const float c_lo = dead_lo ? 1.f : ap_ex2(m_lo - mn_lo), c_hi = dead_hi ? 1.f : ap_ex2(m_hi - mn_hi);
                const float sub_lo = dead_lo ? 0.f : mn_lo, sub_hi = dead_hi ? 0.f : mn_hi;
                float ps_lo = 0.f, ps_hi = 0.f;
                uint32_t pa[2][4][2];
#pragma unroll
                for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float p0 = ap_ex2(fmaf(sc[hh][j][0], scale2, -sub_lo));
                        const float p1 = ap_ex2(fmaf(sc[hh][j][1], scale2, -sub_lo));
                        const float p2 = ap_ex2(fmaf(sc[hh][j][2], scale2, -sub_hi));
                        const float p3 = ap_ex2(fmaf(sc[hh][j][3], scale2, -sub_hi));
                        ps_lo += p0 + p1;
                        ps_hi += p2 + p3;
                        pa[hh][j][0] = ap_pack(p0, p1);
                        pa[hh][j][1] = ap_pack(p2, p3);
                    }
                l_lo = l_lo * c_lo + ps_lo;
                l_hi = l_hi * c_hi + ps_hi;
                m_lo = mn_lo;
                m_hi = mn_hi;
                if (__any_sync(0xffffffffu, c_lo != 1.f || c_hi != 1.f)) {
#pragma unroll
                    for (int i2 = 0; i2 < DT; ++i2) {
                        o[i2][0] *= c_lo;
                        o[i2][1] *= c_lo;
                        o[i2][2] *= c_hi;
                        o[i2][3] *= c_hi;
                    }
                }
                // keys beyond the block's last position lie in the last page only: read zeros for them
                const int live = blk_pos_max + 1 - base;     // keys of this page that were ever written
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
#pragma unroll
                    for (int i2 = 0; i2 < DT; ++i2) {
                        uint4 v = ap_lds128(v_addr + (uint32_t)((8 * i2 * DL_PAGE + 32 * hh) * 2));
                        if (live < DL_PAGE) {
                            uint32_t* wv = reinterpret_cast<uint32_t*>(&v);
                            const int k0 = 32 * hh + 8 * t;
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                if (k0 + 2 * u >= live) wv[u] = 0u;
                                else if (k0 + 2 * u + 1 >= live) wv[u] &= 0x0000ffffu;
                            }
                        }
                        ap_mma(o[i2], pa[hh][0][0], pa[hh][0][1], pa[hh][1][0], pa[hh][1][1], v.x, v.y);
                        ap_mma(o[i2], pa[hh][2][0], pa[hh][2][1], pa[hh][3][0], pa[hh][3][1], v.z, v.w);
                    }
                }
            }
            // The stage may be released only after every MMA fed from it has been issued (an MMA issues
            // when its operands have arrived from shared memory).  The MMAs are not volatile, so pin
            // their results here: the compiler cannot sink them below this point.
#pragma unroll
            for (int i2 = 0; i2 < DT; ++i2) asm volatile("" : "+f"(o[i2][0]), "+f"(o[i2][1]), "+f"(o[i2][2]), "+f"(o[i2][3]));
            // ... and the reads themselves must be done before the copy engine may overwrite the stage:
            // without this fence a slot that was refilled at once showed rows of the new chunk to the old reads.
            __threadfence_block();
            __syncwarp();
            if (lane == 0) ap_mbar_arrive(&empty_bar[s]);
        }

        if (!gave_up) {
            l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
            l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
            l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
            l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
            const float inv_lo = 1.0f / l_lo, inv_hi = 1.0f / l_hi;
            __nv_bfloat16* o_lo = out + (size_t)(tok0 + g) * out_stride + (size_t)h * HD;
            __nv_bfloat16* o_hi = out + (size_t)(tok0 + g + 8) * out_stride + (size_t)h * HD;
#pragma unroll
            for (int i = 0; i < DT; ++i) {
                if (ok_lo) *reinterpret_cast<__nv_bfloat162*>(o_lo + 8 * i + 2 * t) = __floats2bfloat162_rn(o[i][0] * inv_lo, o[i][1] * inv_lo);
                if (ok_hi) *reinterpret_cast<__nv_bfloat162*>(o_hi + 8 * i + 2 * t) = __floats2bfloat162_rn(o[i][2] * inv_hi, o[i][3] * inv_hi);
            }
        }
    }
    __syncthreads();                                         // nobody leaves while copies may still land
}

template <int HD>
static int ap_launch(dim3 grid, cudaStream_t s, const void* q, int q_stride, void* out, int out_stride,
                     const void* k_pool, const void* v_pool, int n_pages, const int32_t* tile_seq,
                     const int32_t* tile_row0, const int32_t* seq_start, const int32_t* seq_new,
                     const int32_t* cu_new, const int32_t* block_table, int bt_stride, int nh, int nkv, float scale,
                     int window, int* status) {
    const size_t smem = (size_t)AP_STAGES * 2 * DL_PAGE * HD * 2;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "attention_prefill: shared memory %zu: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    attention_prefill_kernel<HD><<<grid, AP_THREADS, smem, s>>>(
        (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pool,
        (const __nv_bfloat16*)v_pool, n_pages, tile_seq, tile_row0, seq_start, seq_new, cu_new, block_table, bt_stride,
        nh, nkv, scale, window, status);
    DL_CHECK_LAUNCH("attention_prefill");
    return DL_OK;
}

// q, out: bf16 [T, nh*hd] packed new tokens of all sequences.  tile_seq / tile_row0: for every
// 128-row tile its sequence and its first row among that sequence's new tokens.  seq_start,
// seq_new: cached length before the step and new tokens, per sequence; cu_new: packed offsets.
// status: int32, set non-zero if a wait expired.
extern "C" int dl_attention_prefill_bf16(const void* q, int q_stride, void* out, int out_stride,
                                         const void* k_pool, const void* v_pool, int n_pages,
                                         const int32_t* tile_seq, const int32_t* tile_row0, int n_tiles,
                                         const int32_t* seq_start, const int32_t* seq_new, const int32_t* cu_new,
                                         const int32_t* block_table, int bt_stride, int nh, int nkv, int hd,
                                         float scale, int window, int* status, void* stream) {
    DL_REQUIRE(n_tiles >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0, "attention_prefill: bad sizes");
    DL_REQUIRE(scale > 0.f, "attention_prefill: the score scale must be positive");
    DL_REQUIRE(status != nullptr, "attention_prefill: needs a status word");
    DL_REQUIRE(q_stride % 8 == 0 && out_stride % 2 == 0 && ((uintptr_t)q % 16) == 0 && ((uintptr_t)out % 4) == 0 &&
                   ((uintptr_t)k_pool % 16) == 0 && ((uintptr_t)v_pool % 16) == 0,
               "attention_prefill: q and the pools must be 16-byte aligned");
    DL_REQUIRE(nh <= 65535, "attention_prefill: too many heads");
    if (n_tiles == 0) return DL_OK;
    DL_REQUIRE(n_tiles <= 65535, "attention_prefill: too many tiles (%d)", n_tiles);
    dim3 grid(nh, n_tiles);
    cudaStream_t s = (cudaStream_t)stream;
#define AP_CASE(HDV)                                                                                                  \
    if (hd == HDV)                                                                                                    \
        return ap_launch<HDV>(grid, s, q, q_stride, out, out_stride, k_pool, v_pool, n_pages, tile_seq, tile_row0,     \
                              seq_start, seq_new, cu_new, block_table, bt_stride, nh, nkv, scale, window, status);
    AP_CASE(32) AP_CASE(64) AP_CASE(96) AP_CASE(128)
#undef AP_CASE
    return dl_fail(DL_ERR_UNSUPPORTED, "attention_prefill: head_dim %d (takes 32, 64, 96, 128)", hd);
}
