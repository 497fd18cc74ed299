// Token selection on the device: repetition penalty, greedy argmax, and the sampled chain
// temperature -> top-k -> top-p -> min-p -> categorical draw, one thread block per row.
//
// Semantics follow the reference's host-side samplers:
//   RepetitionPenaltyProcessor.cs:14-55  each distinct recent id once: logit>0 ? /p : *p
//   SamplerPipeline.cs:141-157           processors, argmax if greedy, else steps, then draw
//   TemperatureSampler.cs:22-29          logits *= 1/T, skipped for T == 1
//   TopKSampler.cs:32-79                 keep the k largest; ties at the k-th value admitted in
//                                        index order until exactly k are kept
//   TopPSampler.cs:23-81                 smallest set of most probable tokens reaching p
//   MinPSampler.cs:23-37                 mask logit < max + ln(min_p)
//   CategoricalSampler.cs:18-41          first index whose running probability exceeds r
// (all under src/DotLLM.Engine/Samplers/).
//
// Nothing is sorted.  Thresholds are found by an 8-bit radix descent over order-preserving
// integer keys of the logits, by count for top-k and by probability mass for top-p.  Masses
// are exp(v - max) in float32 converted to 32.32 fixed point and summed as integers, so every
// sum is exact, independent of thread order, and a seeded draw is reproducible bit for bit.
#include "common.cuh"
#include <cooperative_groups.h>

#define SMP_THREADS 1024
#define SMP_ITEMS 4
typedef unsigned long long u64;

__device__ __forceinline__ uint32_t smp_key(float v) {          // ascending float order -> ascending uint
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float smp_unkey(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
__device__ __forceinline__ u64 smp_mass(float v, float vmax) {   // exp(v - vmax) in 32.32 fixed point
    return __float2ull_rn(expf(v - vmax) * 4294967296.0f);
}

template <typename V>
__device__ __forceinline__ V smp_block_sum(V v, V* scratch /* 33 */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        V w = lane < (SMP_THREADS / 32) ? scratch[lane] : (V)0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
        if (lane == 0) scratch[32] = w;
    }
    __syncthreads();
    return scratch[32];
}

// Exclusive prefix sum over the block in thread order; *total receives the block's sum.
template <typename V>
__device__ __forceinline__ V smp_block_scan(V v, V* scratch /* 33 */, V* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    V inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        V n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    __syncthreads();
    if (lane == 31) scratch[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        V w = lane < (SMP_THREADS / 32) ? scratch[lane] : (V)0;
        V winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            V n = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += n;
        }
        scratch[lane] = winc - w;                  // exclusive offset of each warp
        if (lane == 31) scratch[32] = winc;
    }
    __syncthreads();
    *total = scratch[32];
    return scratch[warp] + inc - v;
}

struct SmpShared {
    u64 hist_mass[256];
    unsigned int hist_count[256];
    u64 scratch64[33];
    int scratch32[33];
    float red_val[32];
    int red_idx[32];
    uint32_t prefix;
    u64 above;          // mass or count strictly above the chosen bin
    unsigned int equal;  // elements in the chosen bin (after the last pass: equal to the key)
    int found;
};

// Radix descent.  BY_MASS: find the key at which the mass of keys >= it first reaches
// `target`; else the key with `target` elements at or above it.  Elements below `low_key` are
// ignored; of those equal to low_key only `low_allowed` of `low_equal` count.
template <bool BY_MASS>
__device__ void smp_select(SmpShared& sh, const float* x, int V, float inv_t, float vmax, uint32_t low_key,
                           unsigned int low_allowed, unsigned int low_equal, u64 target, uint32_t* key_out,
                           u64* above_out, unsigned int* equal_out) {
    uint32_t prefix = 0;
    u64 above = 0;
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        for (int b = threadIdx.x; b < 256; b += SMP_THREADS) { sh.hist_mass[b] = 0; sh.hist_count[b] = 0; }
        __syncthreads();
        for (int i = threadIdx.x; i < V; i += SMP_THREADS) {
            float v = x[i] * inv_t;
            if (v != v) v = -INFINITY;
            const uint32_t key = smp_key(v);
            if (key < low_key) continue;
            if (pass > 0 && (key >> (shift + 8)) != prefix) continue;
            const int bin = (key >> shift) & 255;
            atomicAdd(&sh.hist_count[bin], 1u);
            if (BY_MASS) atomicAdd(&sh.hist_mass[bin], smp_mass(v, vmax));
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            // Only `low_allowed` of the `low_equal` elements at low_key take part.
            if (low_equal > low_allowed && (pass == 0 || (low_key >> (shift + 8)) == prefix)) {
                const int bin = (low_key >> shift) & 255;
                sh.hist_count[bin] -= (low_equal - low_allowed);
                if (BY_MASS) sh.hist_mass[bin] -= (u64)(low_equal - low_allowed) * smp_mass(smp_unkey(low_key), vmax);
            }
            int digit = 0;
            u64 cum = above;
            for (int b = 255; b >= 0; --b) {
                const u64 w = BY_MASS ? sh.hist_mass[b] : (u64)sh.hist_count[b];
                if (sh.hist_count[b] != 0 && cum + w >= target) { digit = b; break; }
                cum += w;
                if (b == 0) {                       // target beyond the total: settle on the lowest used bin
                    for (int c = 0; c < 256; ++c)
                        if (sh.hist_count[c] != 0) { digit = c; break; }
                    cum = above;
                    for (int c = 255; c > digit; --c) cum += BY_MASS ? sh.hist_mass[c] : (u64)sh.hist_count[c];
                }
            }
            sh.prefix = (pass == 0 ? 0u : (prefix << 8)) | (uint32_t)digit;
            sh.above = cum;
            sh.equal = sh.hist_count[digit];
        }
        __syncthreads();
        prefix = sh.prefix;
        above = sh.above;
    }
    *key_out = prefix;
    *above_out = above;
    *equal_out = sh.equal;
    __syncthreads();
}

__global__ void __launch_bounds__(SMP_THREADS)
sample_kernel(const float* __restrict__ logits, int row_stride, int V, const float* __restrict__ temperature,
              const int32_t* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ min_p, const float* __restrict__ uniform, int32_t* __restrict__ out) {
    __shared__ SmpShared sh;
    const int row = blockIdx.x;
    const float* x = logits + (size_t)row * row_stride;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float temp = temperature ? temperature[row] : 0.f;
    const float inv_t = (temp > 0.f && temp != 1.0f) ? 1.0f / temp : 1.0f;

    // ---- maximum and its first index (the greedy answer and the softmax shift)
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += SMP_THREADS) {
        float v = x[i] * inv_t;
        if (v != v) v = -INFINITY;
        if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { sh.red_val[warp] = best; sh.red_idx[warp] = best_i; }
    __syncthreads();
    if (warp == 0) {
        best = sh.red_val[lane];
        best_i = sh.red_idx[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        if (lane == 0) { sh.red_val[0] = best; sh.red_idx[0] = best_i; }
    }
    __syncthreads();
    const float vmax = sh.red_val[0];
    const int arg_max = sh.red_idx[0] < V ? sh.red_idx[0] : 0;
    __syncthreads();
    if (!(temp > 0.f) || vmax == -INFINITY) {        // greedy, or nothing finite to draw from
        if (threadIdx.x == 0) out[row] = arg_max;
        return;
    }

    // ---- thresholds: everything above low_key is kept, and `allowed` of the `equal` at it
    uint32_t low_key = 0;
    unsigned int allowed = 0, equal = 0;
    const int k = top_k ? top_k[row] : 0;
    if (k > 0 && k < V) {
        u64 above;
        smp_select<false>(sh, x, V, inv_t, vmax, 0u, 0u, 0u, (u64)k, &low_key, &above, &equal);
        allowed = (unsigned int)((u64)k - above);
        if (allowed > equal) allowed = equal;
    }
    const float p = top_p ? top_p[row] : 1.0f;
    if (p < 1.0f) {
        u64 part = 0;
        for (int i = threadIdx.x; i < V; i += SMP_THREADS) {
            float v = x[i] * inv_t;
            if (v != v) v = -INFINITY;
            if (smp_key(v) > low_key) part += smp_mass(v, vmax);
        }
        u64 z1 = smp_block_sum<u64>(part, sh.scratch64);
        z1 += (u64)allowed * smp_mass(smp_unkey(low_key), vmax);
        double want = ceil((double)p * (double)z1);
        u64 target = want < 1.0 ? 1ull : (u64)want;
        uint32_t key_p;
        u64 above;
        unsigned int equal_p;
        smp_select<true>(sh, x, V, inv_t, vmax, low_key, allowed, equal, target, &key_p, &above, &equal_p);
        const unsigned int avail = equal_p;         // already reduced to `allowed` when key_p == low_key
        const u64 unit = smp_mass(smp_unkey(key_p), vmax);
        unsigned int needed = avail;
        if (unit > 0 && target > above) {
            const u64 n = (target - above + unit - 1) / unit;
            needed = n < (u64)avail ? (unsigned int)n : avail;
        }
        if (needed < 1) needed = 1;
        if (key_p == low_key) {
            // ranks are counted among all `equal` elements at the key; fewer of them are admitted
            allowed = needed;
        } else {
            low_key = key_p;
            allowed = needed;
            equal = equal_p;
        }
    }
    const float mp = min_p ? min_p[row] : 0.f;
    const float floor_v = mp > 0.f ? vmax + logf(mp) : -INFINITY;

    // ---- total kept mass
    u64 part = 0;
    for (int i = threadIdx.x; i < V; i += SMP_THREADS) {
        float v = x[i] * inv_t;
        if (v != v) v = -INFINITY;
        if (smp_key(v) > low_key && !(v < floor_v)) part += smp_mass(v, vmax);
    }
    u64 z = smp_block_sum<u64>(part, sh.scratch64);
    const float low_v = smp_unkey(low_key);
    const bool low_in = low_key != 0 && !(low_v < floor_v);
    if (low_in) z += (u64)allowed * smp_mass(low_v, vmax);
    if (z == 0) {
        if (threadIdx.x == 0) out[row] = arg_max;
        return;
    }
    const float r = uniform ? uniform[row] : 0.f;
    u64 target = (u64)((double)r * (double)z);
    if (target >= z) target = z - 1;

    // ---- walk in index order to the first index whose running mass exceeds the target
    const bool need_rank = low_in && allowed < equal;
    if (threadIdx.x == 0) sh.found = -1;
    __syncthreads();
    u64 run_mass = 0;
    int run_ties = 0;
    for (int base = 0; base < V; base += SMP_THREADS * SMP_ITEMS) {
        float v[SMP_ITEMS];
        uint32_t key[SMP_ITEMS];
        int ties = 0;
#pragma unroll
        for (int e = 0; e < SMP_ITEMS; ++e) {
            const int i = base + threadIdx.x * SMP_ITEMS + e;
            float t = i < V ? x[i] * inv_t : -INFINITY;
            if (t != t) t = -INFINITY;
            v[e] = t;
            key[e] = i < V ? smp_key(t) : 0u;
            if (i < V && key[e] == low_key) ++ties;
        }
        int rank = 0;
        if (need_rank) {
            int total;
            rank = run_ties + smp_block_scan<int>(ties, sh.scratch32, &total);
            run_ties += total;
        }
        u64 m[SMP_ITEMS];
        u64 mine = 0;
#pragma unroll
        for (int e = 0; e < SMP_ITEMS; ++e) {
            const int i = base + threadIdx.x * SMP_ITEMS + e;
            bool keep = false;
            if (i < V) {
                if (key[e] > low_key) keep = !(v[e] < floor_v);
                else if (key[e] == low_key && low_in) {
                    keep = need_rank ? (rank < (int)allowed) : true;
                    ++rank;
                }
            }
            m[e] = keep ? smp_mass(v[e], vmax) : 0ull;
            mine += m[e];
        }
        u64 total;
        u64 before = run_mass + smp_block_scan<u64>(mine, sh.scratch64, &total);
        if (target >= before && target < before + mine) {
#pragma unroll
            for (int e = 0; e < SMP_ITEMS; ++e) {
                if (m[e] != 0 && target >= before && target < before + m[e]) sh.found = base + threadIdx.x * SMP_ITEMS + e;
                before += m[e];
            }
        }
        run_mass += total;
        __syncthreads();
        if (sh.found >= 0) break;
    }
    if (threadIdx.x == 0) out[row] = sh.found >= 0 ? sh.found : arg_max;
}

// One block per row.  `prev` holds generated ids, those of step row r in row row_map[r] (r itself
// without a map), ids [0, prev_len[r]).  With `append_pos`, the block first writes append_token[r] at
// append_pos[r] of its history row (< 0: nothing to write): a caller that keeps the histories on the
// device sends one id per row and step instead of the whole history.  The last `window[r]` of the ids
// (0 = all) are penalised once per distinct id.
__global__ void __launch_bounds__(256)
repetition_penalty_kernel(float* __restrict__ logits, int row_stride, int V, int32_t* __restrict__ prev,
                          int prev_stride, int prev_rows, const int32_t* __restrict__ row_map,
                          const int32_t* __restrict__ append_pos, const int32_t* __restrict__ append_token,
                          const int32_t* __restrict__ prev_len, const float* __restrict__ penalty,
                          const int32_t* __restrict__ window) {
    const int row = blockIdx.x;
    const int hrow = row_map ? row_map[row] : row;
    if (hrow < 0 || hrow >= prev_rows) return;                // host-validated
    int32_t* ids = prev + (size_t)hrow * prev_stride;
    if (append_pos != nullptr) {
        const int at = append_pos[row];
        if (threadIdx.x == 0 && at >= 0 && at < prev_stride) ids[at] = append_token[row];
        __syncthreads();
    }
    const float pen = penalty[row];
    const int n = min(prev_len[row], prev_stride);
    if (pen == 1.0f || n <= 0) return;
    const int w = window[row];
    const int start = (w > 0 && n - w > 0) ? n - w : 0;
    float* x = logits + (size_t)row * row_stride;
    for (int i = start + threadIdx.x; i < n; i += blockDim.x) {
        const int id = ids[i];
        if (id < 0 || id >= V) continue;
        bool first = true;
        for (int j = start; j < i; ++j)
            if (ids[j] == id) { first = false; break; }
        if (!first) continue;
        const float v = x[id];
        x[id] = v > 0.f ? v / pen : v * pen;
    }
}

// Greedy for every row (no temperature given): a cluster of SMP_SPLIT blocks per row, each scanning its
// slice of the vocabulary; block 0 of the cluster then reads the others' (maximum, first index)
// through distributed shared memory.  One block per row reads a 128k-entry row in about 20 us; eight
// share it in about 4.  Same answer as sample_kernel's greedy branch: NaN counts as -inf, the first
// index of the maximum wins, index 0 if nothing is finite.
#define SMP_SPLIT 8
#define AMX_THREADS 512
__global__ void __cluster_dims__(SMP_SPLIT, 1, 1) __launch_bounds__(AMX_THREADS)
argmax_cluster_kernel(const float* __restrict__ logits, int row_stride, int V, int32_t* __restrict__ out) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float red_val[32];
    __shared__ int red_idx[32];
    __shared__ float part_val;
    __shared__ int part_idx;
    const int row = blockIdx.y, part = (int)cluster.block_rank();
    const float* x = logits + (size_t)row * row_stride;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int span = (V + SMP_SPLIT - 1) / SMP_SPLIT;
    const int lo = part * span, hi = min(V, lo + span);
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = lo + (int)threadIdx.x; i < hi; i += AMX_THREADS) {
        float v = x[i];
        if (v != v) v = -INFINITY;
        if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { red_val[warp] = best; red_idx[warp] = best_i; }
    __syncthreads();
    if (warp == 0) {
        best = lane < AMX_THREADS / 32 ? red_val[lane] : -INFINITY;
        best_i = lane < AMX_THREADS / 32 ? red_idx[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        if (lane == 0) { part_val = best; part_idx = best_i; }
    }
    cluster.sync();                                          // every block's answer is in its shared memory
    if (part == 0 && warp == 0) {
        best = -INFINITY;
        best_i = 0x7fffffff;
        if (lane < SMP_SPLIT) {
            best = *cluster.map_shared_rank(&part_val, lane);
            best_i = *cluster.map_shared_rank(&part_idx, lane);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        if (lane == 0) out[row] = best_i < V ? best_i : 0;
    }
    cluster.sync();                                          // nobody leaves while block 0 may still read it
}

// The sampled chain with a row shared by a cluster of SMP_SPLIT blocks.  One block per row walks the
// row's logits a dozen times from global memory (about 40 us a pass over 128k entries: 130 us for a
// plain temperature draw, 400 us with top-k and top-p); here each block keeps its slice of the scaled
// row in shared memory, every pass runs over shared memory, and what the passes need of each other
// (maxima, histograms, masses) is read from the other blocks' shared memory.  Every sum is of integers
// (counts and fixed-point masses), so the token is the one sample_kernel gives, bit for bit.
#define SC_THREADS 512
#define SC_ITEMS 4
struct ScShared {
    u64 hist_mass[2][256];              // this block's histograms of this pass and the one before (peers read them)
    unsigned int hist_count[2][256];
    u64 top_count[4], top_mass[4];      // this block's sums of the four highest bins of a first digit (peers read them)
    u64 tot_mass[256];                  // the row's histogram, summed over the cluster
    unsigned int tot_count[256];
    u64 scratch64[33];
    int scratch32[33];
    float red_val[32];
    int red_idx[32];
    float part_val;                     // this block's maximum and its first index (peers read them)
    int part_idx;
    u64 part_sum[4];                    // this block's sums, one slot per phase that needs one (peers read them)
    unsigned int part_ties;
    uint32_t prefix;
    u64 above;
    unsigned int equal;
    int found;
};

template <typename V>
__device__ __forceinline__ V sc_block_sum(V v, V* scratch /* 33 */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        V w = lane < (SC_THREADS / 32) ? scratch[lane] : (V)0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
        if (lane == 0) scratch[32] = w;
    }
    __syncthreads();
    return scratch[32];
}
template <typename V>
__device__ __forceinline__ V sc_block_scan(V v, V* scratch /* 33 */, V* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    V inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        V n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    __syncthreads();
    if (lane == 31) scratch[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        V w = lane < (SC_THREADS / 32) ? scratch[lane] : (V)0;
        V winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            V n = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += n;
        }
        scratch[lane] = winc - w;
        if (lane == 31) scratch[32] = winc;
    }
    __syncthreads();
    *total = scratch[32];
    return scratch[warp] + inc - v;
}

// The block's sum `mine` (already summed over the block, the same in every thread) added over the
// cluster in rank order, through slot `which` of part_sum.  A slot is used once per launch, so one
// cluster barrier (write -> read) is enough.
__device__ __forceinline__ u64 sc_cluster_sum(cooperative_groups::cluster_group& cluster, ScShared& sh, int which, u64 mine,
                                              u64* before_me) {
    if (threadIdx.x == 0) sh.part_sum[which] = mine;
    cluster.sync();
    u64 total = 0, before = 0;
    const int me = (int)cluster.block_rank();
    for (int r = 0; r < SMP_SPLIT; ++r) {
        const u64 v = *cluster.map_shared_rank(&sh.part_sum[which], r);
        if (r < me) before += v;
        total += v;
    }
    if (before_me) *before_me = before;
    return total;
}

// smp_select over a row whose slices lie in the cluster's shared memories (`sv`: this block's n values).
// The first digit is found without a histogram where it can be: of the top byte of the keys only a
// handful of values occur (sign and seven exponent bits), so a histogram's atomic additions would pile
// up on a few addresses.  Every thread instead sums, in registers, the four highest bins that can be
// occupied (from the bin of the row's maximum down) and everything below them as one; if the target
// falls into those four, as it does unless nearly the whole row is kept, that is the digit.  Otherwise,
// and for the three digits below, histograms in shared memory are summed over the cluster; two sets of
// them alternate (`epoch` counts the passes of a launch), so one cluster barrier a pass is enough.
template <bool BY_MASS>
__device__ void sc_select(cooperative_groups::cluster_group& cluster, ScShared& sh, int& epoch, const float* sv, int n,
                          float vmax, uint32_t low_key, unsigned int low_allowed, unsigned int low_equal, u64 target,
                          uint32_t* key_out, u64* above_out, unsigned int* equal_out) {
    uint32_t prefix = 0;
    u64 above = 0;
    unsigned int equal = 0;
    int pass0 = 0;
    {
        const int top = (int)(smp_key(vmax) >> 24);
        unsigned int c0 = 0, c1 = 0, c2 = 0, c3 = 0;
        u64 m0 = 0, m1 = 0, m2 = 0, m3 = 0;
        for (int i = threadIdx.x; i < n; i += SC_THREADS) {
            const float v = sv[i];
            const uint32_t key = smp_key(v);
            if (key < low_key) continue;
            const int d = top - (int)(key >> 24);
            if (d > 3) continue;
            const u64 m = BY_MASS ? smp_mass(v, vmax) : 0ull;
            if (d == 0) { ++c0; m0 += m; }
            else if (d == 1) { ++c1; m1 += m; }
            else if (d == 2) { ++c2; m2 += m; }
            else { ++c3; m3 += m; }
        }
        // counts and masses of the four bins, summed over the block, then over the cluster
        const u64 bc[4] = {sc_block_sum<u64>((u64)c0, sh.scratch64), sc_block_sum<u64>((u64)c1, sh.scratch64),
                           sc_block_sum<u64>((u64)c2, sh.scratch64), sc_block_sum<u64>((u64)c3, sh.scratch64)};
        u64 bm[4] = {0, 0, 0, 0};
        if (BY_MASS) {
            bm[0] = sc_block_sum<u64>(m0, sh.scratch64);
            bm[1] = sc_block_sum<u64>(m1, sh.scratch64);
            bm[2] = sc_block_sum<u64>(m2, sh.scratch64);
            bm[3] = sc_block_sum<u64>(m3, sh.scratch64);
        }
        if (threadIdx.x == 0) {
            for (int j = 0; j < 4; ++j) { sh.top_count[j] = bc[j]; sh.top_mass[j] = bm[j]; }
        }
        cluster.sync();
        u64 tc[4] = {0, 0, 0, 0}, tm[4] = {0, 0, 0, 0};
        for (int r = 0; r < SMP_SPLIT; ++r) {
            const ScShared* peer = cluster.map_shared_rank(&sh, r);
            for (int j = 0; j < 4; ++j) {
                tc[j] += peer->top_count[j];
                if (BY_MASS) tm[j] += peer->top_mass[j];
            }
        }
        if (low_equal > low_allowed) {                      // only `low_allowed` of the `low_equal` elements at low_key take part
            const int d = top - (int)(low_key >> 24);
            if (d >= 0 && d <= 3) {
                tc[d] -= (low_equal - low_allowed);
                if (BY_MASS) tm[d] -= (u64)(low_equal - low_allowed) * smp_mass(smp_unkey(low_key), vmax);
            }
        }
        u64 cum = 0;
        for (int j = 0; j < 4 && !pass0; ++j) {              // the same in every thread of every block
            const u64 w = BY_MASS ? tm[j] : tc[j];
            if (tc[j] != 0 && cum + w >= target) {
                prefix = (uint32_t)(top - j);
                above = cum;
                equal = (unsigned int)tc[j];
                pass0 = 1;
            } else {
                cum += w;
            }
        }
    }
    for (int pass = pass0; pass < 4; ++pass, ++epoch) {
        const int shift = 24 - 8 * pass;
        u64* hist_mass = sh.hist_mass[epoch & 1];
        unsigned int* hist_count = sh.hist_count[epoch & 1];
        for (int b = threadIdx.x; b < 256; b += SC_THREADS) { hist_mass[b] = 0; hist_count[b] = 0; }
        __syncthreads();
        for (int i = threadIdx.x; i < n; i += SC_THREADS) {
            const float v = sv[i];
            const uint32_t key = smp_key(v);
            if (key < low_key) continue;
            if (pass > 0 && (key >> (shift + 8)) != prefix) continue;
            const int bin = (key >> shift) & 255;
            atomicAdd(&hist_count[bin], 1u);
            if (BY_MASS) atomicAdd(&hist_mass[bin], smp_mass(v, vmax));
        }
        cluster.sync();                                      // every block's histogram of this pass is complete
        for (int b = threadIdx.x; b < 256; b += SC_THREADS) {
            unsigned int c = 0;
            u64 m = 0;
            for (int r = 0; r < SMP_SPLIT; ++r) {
                const ScShared* peer = cluster.map_shared_rank(&sh, r);
                c += peer->hist_count[epoch & 1][b];
                if (BY_MASS) m += peer->hist_mass[epoch & 1][b];
            }
            sh.tot_count[b] = c;
            sh.tot_mass[b] = m;
        }
        __syncthreads();
        if (threadIdx.x == 0 && low_equal > low_allowed && (pass == 0 || (low_key >> (shift + 8)) == prefix)) {
            const int bin = (low_key >> shift) & 255;
            sh.tot_count[bin] -= (low_equal - low_allowed);
            if (BY_MASS) sh.tot_mass[bin] -= (u64)(low_equal - low_allowed) * smp_mass(smp_unkey(low_key), vmax);
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            // The digit: from bin 255 down, the first used bin at which the running sum reaches the target.
            // Lane l looks at bins 8l .. 8l+7; the lanes above it hold what lies before them.
            const int l = threadIdx.x;
            u64 w[8];
            unsigned int cnt[8];
            u64 mine = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                cnt[j] = sh.tot_count[8 * l + j];
                w[j] = BY_MASS ? sh.tot_mass[8 * l + j] : (u64)cnt[j];
                mine += w[j];
            }
            u64 before = mine;                               // inclusive sum over lanes l .. 31
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const u64 up = __shfl_down_sync(0xffffffffu, before, o);
                if (l + o < 32) before += up;
            }
            const u64 all = __shfl_sync(0xffffffffu, before, 0);
            u64 cum = above + before - mine;                 // what lies in the bins above this lane's
            int digit = -1;
            u64 cum_at = 0;
#pragma unroll
            for (int j = 7; j >= 0; --j) {
                if (digit < 0 && cnt[j] != 0 && cum + w[j] >= target) { digit = 8 * l + j; cum_at = cum; }
                cum += w[j];
            }
            const unsigned hit = __ballot_sync(0xffffffffu, digit >= 0);
            int lowest_used = 256;
#pragma unroll
            for (int j = 7; j >= 0; --j)
                if (cnt[j] != 0) lowest_used = 8 * l + j;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) lowest_used = min(lowest_used, __shfl_xor_sync(0xffffffffu, lowest_used, o));
            if (hit) {
                const int src = 31 - __clz(hit);
                digit = __shfl_sync(0xffffffffu, digit, src);
                cum_at = __shfl_sync(0xffffffffu, cum_at, src);
            } else {                                         // target beyond the total: settle on the lowest used bin
                digit = lowest_used < 256 ? lowest_used : 0;
                u64 at_or_below = 0;                         // what lies in bins <= digit
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (8 * l + j <= digit) at_or_below += w[j];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) at_or_below += __shfl_xor_sync(0xffffffffu, at_or_below, o);
                cum_at = above + all - at_or_below;
            }
            if (l == 0) {
                sh.prefix = (pass == 0 ? 0u : (prefix << 8)) | (uint32_t)digit;
                sh.above = cum_at;
                sh.equal = sh.tot_count[digit];
            }
        }
        __syncthreads();
        prefix = sh.prefix;
        above = sh.above;
        equal = sh.equal;
    }
    *key_out = prefix;
    *above_out = above;
    *equal_out = equal;
    __syncthreads();
}

__global__ void __cluster_dims__(SMP_SPLIT, 1, 1) __launch_bounds__(SC_THREADS)
sample_cluster_kernel(const float* __restrict__ logits, int row_stride, int V, int span, const float* __restrict__ temperature,
                      const int32_t* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
                      const float* __restrict__ uniform, int32_t* __restrict__ out) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    extern __shared__ __align__(16) float sc_values[];       // this block's slice of the row, scaled, NaN as -inf
    __shared__ ScShared sh;
    const int row = blockIdx.y, part = (int)cluster.block_rank();
    const float* x = logits + (size_t)row * row_stride;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float temp = temperature[row];
    const float inv_t = (temp > 0.f && temp != 1.0f) ? 1.0f / temp : 1.0f;
    const int lo = min(V, part * span), n = min(V, lo + span) - lo;

    // ---- the slice into shared memory; maximum and its first index
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += SC_THREADS) {
        float v = x[lo + i] * inv_t;
        if (v != v) v = -INFINITY;
        sc_values[i] = v;
        if (v > best || (v == best && lo + i < best_i)) { best = v; best_i = lo + i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { sh.red_val[warp] = best; sh.red_idx[warp] = best_i; }
    __syncthreads();
    if (warp == 0) {
        best = lane < SC_THREADS / 32 ? sh.red_val[lane] : -INFINITY;
        best_i = lane < SC_THREADS / 32 ? sh.red_idx[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        if (lane == 0) { sh.part_val = best; sh.part_idx = best_i; }
    }
    cluster.sync();                                          // every block's slice and maximum are in place
    best = -INFINITY;
    best_i = 0x7fffffff;
    for (int r = 0; r < SMP_SPLIT; ++r) {                    // every thread reads all eight: the same answer everywhere
        const float ov = *cluster.map_shared_rank(&sh.part_val, r);
        const int oi = *cluster.map_shared_rank(&sh.part_idx, r);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    const float vmax = best;
    const int arg_max = best_i < V ? best_i : 0;
    if (!(temp > 0.f) || vmax == -INFINITY) {                // greedy, or nothing finite to draw from: the same in every block
        if (part == 0 && threadIdx.x == 0) out[row] = arg_max;
        cluster.sync();                                      // nobody leaves while a peer may still read its maximum
        return;
    }
    const float* sv = sc_values;
    int epoch = 0;                                           // histogram passes so far

    // ---- thresholds: everything above low_key is kept, and `allowed` of the `equal` at it
    uint32_t low_key = 0;
    unsigned int allowed = 0, equal = 0;
    const int k = top_k ? top_k[row] : 0;
    if (k > 0 && k < V) {
        u64 above;
        sc_select<false>(cluster, sh, epoch, sv, n, vmax, 0u, 0u, 0u, (u64)k, &low_key, &above, &equal);
        allowed = (unsigned int)((u64)k - above);
        if (allowed > equal) allowed = equal;
    }
    const float p = top_p ? top_p[row] : 1.0f;
    if (p < 1.0f) {
        u64 part_mass = 0;
        for (int i = threadIdx.x; i < n; i += SC_THREADS)
            if (smp_key(sv[i]) > low_key) part_mass += smp_mass(sv[i], vmax);
        u64 z1 = sc_cluster_sum(cluster, sh, 0, sc_block_sum<u64>(part_mass, sh.scratch64), nullptr);
        z1 += (u64)allowed * smp_mass(smp_unkey(low_key), vmax);
        double want = ceil((double)p * (double)z1);
        u64 target = want < 1.0 ? 1ull : (u64)want;
        uint32_t key_p;
        u64 above;
        unsigned int equal_p;
        sc_select<true>(cluster, sh, epoch, sv, n, vmax, low_key, allowed, equal, target, &key_p, &above, &equal_p);
        const unsigned int avail = equal_p;
        const u64 unit = smp_mass(smp_unkey(key_p), vmax);
        unsigned int needed = avail;
        if (unit > 0 && target > above) {
            const u64 nn = (target - above + unit - 1) / unit;
            needed = nn < (u64)avail ? (unsigned int)nn : avail;
        }
        if (needed < 1) needed = 1;
        if (key_p == low_key) {
            allowed = needed;
        } else {
            low_key = key_p;
            allowed = needed;
            equal = equal_p;
        }
    }
    const float mp = min_p ? min_p[row] : 0.f;
    const float floor_v = mp > 0.f ? vmax + logf(mp) : -INFINITY;
    const float low_v = smp_unkey(low_key);
    const bool low_in = low_key != 0 && !(low_v < floor_v);
    const bool need_rank = low_in && allowed < equal;

    // ---- this slice's kept mass above the threshold and its elements at the threshold, then the row's
    u64 part_mass = 0;
    unsigned int part_ties = 0;
    for (int i = threadIdx.x; i < n; i += SC_THREADS) {
        const float v = sv[i];
        const uint32_t key = smp_key(v);
        if (key > low_key && !(v < floor_v)) part_mass += smp_mass(v, vmax);
        if (key == low_key) ++part_ties;
    }
    const u64 my_above = sc_block_sum<u64>(part_mass, sh.scratch64);
    const u64 my_ties = sc_block_sum<u64>((u64)part_ties, sh.scratch64);
    u64 ties_before = 0, above_before = 0;
    const u64 z_above = sc_cluster_sum(cluster, sh, 1, my_above, &above_before);
    sc_cluster_sum(cluster, sh, 2, my_ties, &ties_before);
    u64 z = z_above;
    if (low_in) z += (u64)allowed * smp_mass(low_v, vmax);
    if (z == 0) {
        if (part == 0 && threadIdx.x == 0) out[row] = arg_max;
        cluster.sync();
        return;
    }
    const float r = uniform[row];
    u64 target = (u64)((double)r * (double)z);
    if (target >= z) target = z - 1;

    // ---- the mass that lies before this slice in index order: what is above the threshold in the slices
    // before, and those of the first `allowed` elements at the threshold that the slices before hold
    const u64 unit_low = low_in ? smp_mass(low_v, vmax) : 0ull;
    const u64 ties_kept_before = need_rank ? (ties_before < (u64)allowed ? ties_before : (u64)allowed) : ties_before;
    const u64 ties_kept_here = need_rank ? ((ties_before + my_ties < (u64)allowed ? ties_before + my_ties : (u64)allowed) - ties_kept_before)
                                         : my_ties;
    const u64 mass_before = above_before + (low_in ? ties_kept_before * unit_low : 0ull);
    const u64 mass_here = my_above + (low_in ? ties_kept_here * unit_low : 0ull);
    const bool mine = target >= mass_before && target < mass_before + mass_here;   // exactly one block of the cluster
    if (mine) {
        // ---- walk this slice in index order to the first index whose running mass exceeds the target
        if (threadIdx.x == 0) sh.found = -1;
        __syncthreads();
        u64 run_mass = mass_before;
        int run_ties = (int)ties_before;
        for (int base = 0; base < n; base += SC_THREADS * SC_ITEMS) {
            float v[SC_ITEMS];
            uint32_t key[SC_ITEMS];
            int ties = 0;
#pragma unroll
            for (int e = 0; e < SC_ITEMS; ++e) {
                const int i = base + threadIdx.x * SC_ITEMS + e;
                v[e] = i < n ? sv[i] : -INFINITY;
                key[e] = i < n ? smp_key(v[e]) : 0u;
                if (i < n && key[e] == low_key) ++ties;
            }
            int rank = 0;
            if (need_rank) {
                int total;
                rank = run_ties + sc_block_scan<int>(ties, sh.scratch32, &total);
                run_ties += total;
            }
            u64 m[SC_ITEMS];
            u64 own = 0;
#pragma unroll
            for (int e = 0; e < SC_ITEMS; ++e) {
                const int i = base + threadIdx.x * SC_ITEMS + e;
                bool keep = false;
                if (i < n) {
                    if (key[e] > low_key) keep = !(v[e] < floor_v);
                    else if (key[e] == low_key && low_in) {
                        keep = need_rank ? (rank < (int)allowed) : true;
                        ++rank;
                    }
                }
                m[e] = keep ? smp_mass(v[e], vmax) : 0ull;
                own += m[e];
            }
            u64 total;
            u64 before = run_mass + sc_block_scan<u64>(own, sh.scratch64, &total);
            if (target >= before && target < before + own) {
#pragma unroll
                for (int e = 0; e < SC_ITEMS; ++e) {
                    if (m[e] != 0 && target >= before && target < before + m[e]) sh.found = lo + base + threadIdx.x * SC_ITEMS + e;
                    before += m[e];
                }
            }
            run_mass += total;
            __syncthreads();
            if (sh.found >= 0) break;
        }
        if (threadIdx.x == 0) out[row] = sh.found >= 0 ? sh.found : arg_max;
    }
    cluster.sync();                                          // nobody leaves while a peer may still read its sums
}

// logits: float32 [rows, V] rows row_stride apart.  temperature/top_k/top_p/min_p/uniform: one
// value per row (NULL = greedy / off).  out: int32 [rows].
// mode: 0 chooses; 1 one block per row; 2 a cluster of blocks per row (refused if the row does not fit).
extern "C" int dl_sample(const float* logits, int row_stride, int rows, int V, const float* temperature,
                         const int32_t* top_k, const float* top_p, const float* min_p, const float* uniform,
                         int32_t* out, int mode, void* stream) {
    DL_REQUIRE(mode >= 0 && mode <= 2, "sample: mode %d", mode);
    DL_REQUIRE(rows >= 0 && V > 0 && row_stride >= V, "sample: bad sizes rows=%d V=%d", rows, V);
    DL_REQUIRE(temperature == nullptr || uniform != nullptr, "sample: a sampled draw needs uniform numbers");
    if (rows == 0) return DL_OK;
    if (temperature == nullptr && rows <= 65535) {
        argmax_cluster_kernel<<<dim3(SMP_SPLIT, rows), AMX_THREADS, 0, (cudaStream_t)stream>>>(logits, row_stride, V, out);
        DL_CHECK_LAUNCH("sample (greedy)");
        return DL_OK;
    }
    // A cluster per row when the rows are long enough for the passes over global memory to matter; its
    // slice must fit a block's shared memory.
    int span = (V + SMP_SPLIT - 1) / SMP_SPLIT;
    span = (span + 3) & ~3;
    const size_t slice_bytes = (size_t)span * sizeof(float);
    const bool fits = slice_bytes <= 160 * 1024 && rows <= 65535;
    const bool split = mode == 2 || (mode == 0 && fits && V >= 8192);
    if (mode == 2 && !fits) return dl_fail(DL_ERR_UNSUPPORTED, "sample: a row of %d values does not fit a cluster's shared memory", V);
    if (split && temperature != nullptr) {
        static size_t configured = 0;
        if (configured < slice_bytes) {
            cudaError_t e = cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)slice_bytes);
            if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "sample: shared memory %zu: %s", slice_bytes, cudaGetErrorString(e));
            configured = slice_bytes;
        }
        sample_cluster_kernel<<<dim3(SMP_SPLIT, rows), SC_THREADS, slice_bytes, (cudaStream_t)stream>>>(
            logits, row_stride, V, span, temperature, top_k, top_p, min_p, uniform, out);
        DL_CHECK_LAUNCH("sample (cluster)");
        return DL_OK;
    }
    sample_kernel<<<rows, SMP_THREADS, 0, (cudaStream_t)stream>>>(logits, row_stride, V, temperature, top_k, top_p,
                                                                 min_p, uniform, out);
    DL_CHECK_LAUNCH("sample");
    return DL_OK;
}

// prev: int32 [prev_rows, prev_stride]; row_map, append_pos, append_token: int32 [rows] or NULL (see the kernel).
extern "C" int dl_repetition_penalty(float* logits, int row_stride, int rows, int V, int32_t* prev, int prev_stride, int prev_rows,
                                     const int32_t* row_map, const int32_t* append_pos, const int32_t* append_token,
                                     const int32_t* prev_len, const float* penalty, const int32_t* window, void* stream) {
    DL_REQUIRE(rows >= 0 && V > 0 && row_stride >= V && prev_stride >= 0 && prev_rows >= 0, "repetition_penalty: bad sizes");
    DL_REQUIRE(row_map != nullptr || prev_rows >= rows, "repetition_penalty: %d rows of history for %d rows", prev_rows, rows);
    DL_REQUIRE((append_pos == nullptr) == (append_token == nullptr), "repetition_penalty: a position and an id to append go together");
    if (rows == 0 || prev_stride == 0) return DL_OK;
    repetition_penalty_kernel<<<rows, 256, 0, (cudaStream_t)stream>>>(logits, row_stride, V, prev, prev_stride, prev_rows, row_map,
                                                                     append_pos, append_token, prev_len, penalty, window);
    DL_CHECK_LAUNCH("repetition_penalty");
    return DL_OK;
}
