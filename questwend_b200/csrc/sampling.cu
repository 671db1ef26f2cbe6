// Sampling on the device in the reference's order (core/sampler.cpp:38-109): penalties over the
// recent tokens; greedy if the temperature is <= 0 (the lowest id wins a tie); else top-k by logit,
// softmax with temperature, top-p (the smallest descending prefix whose share reaches top_p), and
// one draw.  The draw walks the kept tokens in id order with a uniform number from a counter-based
// generator (Philox 4x32-10) keyed by the seed, the sequence's own index and the step, so a
// sequence's tokens do not depend on what else is in the batch.
//
// The general way (sample_kernel, one block per row): nothing is sorted.  The k-th largest logit
// and the top-p cut are found by radix selection over an order-preserving 32-bit key of the logit
// (four passes of 8 bits with a histogram of counts or of probability mass in shared memory); ties
// at a cut are broken toward the lower token id.  Every warp fills a histogram of its own, and the
// lanes of a warp that hit the same bin are added up by one of them first, so no two threads ever
// write the same word and no atomic operation is needed: with a vocabulary of 150,000 a histogram
// shared by the block, updated atomically, cost a millisecond a cut.  Rows are read 16 bytes a load.
//
// The short way, when few tokens can be left (a top-k of at most 1,024, the reference's default
// being 40; or top-p alone, tried as a top-k of 1,024 whose share is of the whole row's mass): the
// pass that finds the maximum also counts the tokens by the top bits of their key; the tokens from
// the bin of the k-th largest key up (at most 8,192) are gathered into shared memory, and the exact
// cut, its ties, top-p and the draw are settled there.  If they do not fit, or top-p needs more than
// the 1,024 tokens, the general way runs.
//
// With few rows (at least 16 chunks of a row find an SM) the two passes of the short way are kernels
// of their own over chunks of a row (sample_scan_kernel, sample_gather_kernel), and sample_kernel
// starts from what they gathered; temperature alone uses them too: the chunks' masses say which
// chunk holds the drawn point, and only that chunk is walked.
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ uint32_t order_key(float x) {
    const uint32_t u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ void philox_round(uint32_t* c, uint32_t k0, uint32_t k1) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

// A uniform number in (0, 1) for (seed, sequence, step).
__device__ double philox_uniform(unsigned long long seed, unsigned int sequence, unsigned int step) {
    uint32_t c[4] = {step, sequence, 0x51574232u, 0u};
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    for (int r = 0; r < 10; ++r) {
        philox_round(c, k0, k1);
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    const unsigned long long bits = ((unsigned long long)c[0] << 21) ^ (unsigned long long)c[1];   // 53 bits
    return ((double)(bits & ((1ull << 53) - 1)) + 0.5) / 9007199254740992.0;
}

struct Cut {            // tokens kept: key > key_cut, or key == key_cut and id <= id_limit
    uint32_t key;
    int id_limit;
};

__device__ __forceinline__ bool kept(const Cut& c, uint32_t key, int id) {
    return key > c.key || (key == c.key && id <= c.id_limit);
}

#define SAMPLE_WARPS (SAMPLE_THREADS / 32)

// Calls f(id, logit, valid) for the whole row.  All threads of the block make the same number of calls (valid is false
// where a thread has no token), so f may use warp-wide operations.  16-byte loads where the row's address allows.
template <typename F>
__device__ __forceinline__ void for_each_logit(const float* row, int V, F f) {
    const int tid = threadIdx.x, nthreads = blockDim.x;
    int done = 0;
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
        const float4* row4 = reinterpret_cast<const float4*>(row);
        const int n4 = V >> 2;
#pragma unroll 2
        for (int base = 0; base < n4; base += nthreads) {
            const int idx = base + tid;
            const bool valid = idx < n4;
            const float4 v = valid ? row4[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
            f(4 * idx, v.x, valid);
            f(4 * idx + 1, v.y, valid);
            f(4 * idx + 2, v.z, valid);
            f(4 * idx + 3, v.w, valid);
        }
        done = n4 << 2;
    }
    for (int base = done; base < V; base += nthreads) {
        const int i = base + tid;
        const bool valid = i < V;
        f(i, valid ? row[i] : 0.f, valid);
    }
}

// A double summed over the block, the warps' sums added in warp order (every thread gets the total).
__device__ double block_sum(double s, double* red_d) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    __syncthreads();
    if (lane == 0) red_d[warp] = s;
    __syncthreads();
    double total = 0.0;
    for (int w = 0; w < (blockDim.x >> 5); ++w) total += red_d[w];
    return total;
}

// Counts by bin, the highest bins first: the bin in which the running count (from `above` on) reaches k, the count before
// that bin and the bin's own; bin 0 if it never does.  For one whole warp: lane l looks at the PER_LANE bins from
// 32 PER_LANE - 1 - PER_LANE l downwards.
template <int PER_LANE>
__device__ void find_count_bin(const int* hist_n, int above, int k, int* out_bin, int* out_above, int* out_at) {
    const int lane = threadIdx.x & 31, top = 32 * PER_LANE - 1 - PER_LANE * lane;
    int local = 0;
    for (int j = 0; j < PER_LANE; ++j) local += hist_n[top - j];
    int incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    const int before = above + incl - local;
    const unsigned crossing = __ballot_sync(0xffffffffu, before < k && before + local >= k);
    const int owner = crossing ? __ffs(crossing) - 1 : 31;
    if (lane == owner) {
        int run = before, j = 0;
        for (; j < PER_LANE - 1 && run + hist_n[top - j] < k; ++j) run += hist_n[top - j];
        if (!crossing) { j = PER_LANE - 1; run = before + local - hist_n[top - j]; }   // never reached: bin 0, the others above it
        *out_bin = top - j;
        *out_above = run;
        *out_at = hist_n[top - j];
    }
}

// Radix selection.  Among the tokens kept by `within`, finds the cut such that the kept
// tokens above it, plus as many tokens at it as needed (lowest ids first), reach `target`:
// a count (by_mass = false) or a probability mass (by_mass = true; mass of token i is
// exp((l_i - lmax) / temperature)).  whist / whist_n: [warps][256], a histogram per warp.
__device__ Cut radix_cut(const float* row, int V, const Cut within, bool by_mass, double target,
                         float lmax, float inv_temp, double* whist, int* whist_n, double* hist, int* hist_n,
                         double* sh_above, uint32_t* sh_prefix) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    double* my_hist = whist + warp * 256;
    int* my_n = whist_n + warp * 256;
    uint32_t prefix = 0, mask = 0;
    double above = 0.0;
    int n_at = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = tid; i < SAMPLE_WARPS * 256; i += blockDim.x) { whist[i] = 0.0; whist_n[i] = 0; }
        __syncthreads();
        for_each_logit(row, V, [&](int i, float l, bool valid) {
            const uint32_t key = order_key(l);
            const bool hit = valid && (key & mask) == prefix && kept(within, key, i);
            const unsigned hits = __ballot_sync(0xffffffffu, hit);
            if (hits == 0u) return;                                   // the same for the whole warp
            if (hit) {
                const int bin = (key >> shift) & 255;
                const unsigned peers = __match_any_sync(hits, bin);  // the lanes that hit this bin
                double sum = (double)__popc(peers);
                if (by_mass) {                                        // their masses, added in lane order
                    const double m = (double)expf((l - lmax) * inv_temp);
                    sum = 0.0;
                    for (unsigned rest = peers; rest; rest &= rest - 1) sum += __shfl_sync(peers, m, __ffs(rest) - 1);
                }
                if (lane == __ffs(peers) - 1) {                       // one lane per bin: no two write the same word
                    my_hist[bin] += sum;
                    my_n[bin] += __popc(peers);
                }
            }
            __syncwarp();                                             // the next call may have another lane write this bin
        });
        __syncthreads();
        for (int bin = tid; bin < 256; bin += blockDim.x) {          // the warps' histograms, added in warp order
            double sum = 0.0;
            int n = 0;
            for (int w = 0; w < SAMPLE_WARPS; ++w) { sum += whist[w * 256 + bin]; n += whist_n[w * 256 + bin]; }
            hist[bin] = sum;
            hist_n[bin] = n;
        }
        __syncthreads();
        if (tid == 0) {
            double run = above;
            int chosen = -1, lowest = -1;
            for (int bin = 255; bin >= 0; --bin) {
                if (hist_n[bin] == 0) continue;
                lowest = bin;
                if (run + hist[bin] >= target) { chosen = bin; break; }
                run += hist[bin];
            }
            if (chosen < 0) { chosen = lowest; run -= hist[lowest]; }     // rounding left the total short: keep all
            *sh_above = run;
            *sh_prefix = prefix | ((uint32_t)chosen << shift);
            hist_n[0] = hist_n[chosen];
            hist[0] = hist[chosen];
        }
        __syncthreads();
        above = *sh_above;
        prefix = *sh_prefix;
        mask |= 255u << shift;
        n_at = hist_n[0];
        __syncthreads();
    }
    // tokens at the cut: how many are needed
    Cut cut;
    cut.key = prefix;
    cut.id_limit = V;
    const double at_mass = hist[0];                // mass (or count) of all tokens at the cut
    __syncthreads();
    long long needed;
    if (by_mass) {
        const double each = at_mass / (double)n_at;
        needed = (long long)ceil((target - above) / each);
    } else {
        needed = (long long)(target - above + 0.5);
    }
    if (needed < 1) needed = 1;
    if (needed < n_at) {                           // a tie across the cut: lowest ids first
        if (tid == 0) {
            int seen = 0, limit = V;
            for (int i = 0; i < V; ++i) {
                const uint32_t key = order_key(row[i]);
                if (key == prefix && kept(within, key, i) && ++seen == needed) { limit = i; break; }
            }
            *(int*)sh_prefix = limit;
        }
        __syncthreads();
        cut.id_limit = *(int*)sh_prefix;
        __syncthreads();
    }
    if (cut.key == within.key && within.id_limit < cut.id_limit) cut.id_limit = within.id_limit;
    return cut;
}

#define SAMPLE_CAND_MAX 8192        // tokens that the small top-k path gathers at most
#define SPLIT_THREADS 256
#define SPLIT_WARPS (SPLIT_THREADS / 32)
#define SPLIT_BITS 10               // the split kernels count the tokens by the top 10 bits of their key
#define SPLIT_BINS (1 << SPLIT_BITS)

// What the split kernels leave for a row, for the sampling kernel to go on from (count null: it scans the row itself).
struct Gathered {
    const float* best;      // [B] the row's maximum
    const int* best_i;      // [B] its id, the lowest among equals
    const int* info;        // [B][4]: the top SPLIT_BITS bits of the k-th largest key, the tokens above those, 1 if they did not fit
    int* count;             // [B] tokens gathered; the sampling kernel sets it back to 0
    int* hist;              // [B][SPLIT_BINS] the row's counts; the sampling kernel sets them back to 0
    const int* id;          // [B][SAMPLE_CAND_MAX]
    const float* logit;     // [B][SAMPLE_CAND_MAX]
    const double* mass;     // [B][n_chunks] the chunks' sums of exp((l - best) / temperature) over all their tokens, or null
    int n_chunks, chunk;    // chunks a row, tokens a chunk
};

// Penalties over the recent tokens, each distinct token once, for the tokens in [i0, i1) of the row.
__device__ void apply_penalties(float* row, int i0, int i1, const int* rec, int window, float repeat_penalty,
                                float presence_penalty, float frequency_penalty) {
    for (int i = threadIdx.x; i < window; i += blockDim.x) {
        const int tok = rec[i];
        if (tok < i0 || tok >= i1) continue;
        bool first = true;
        for (int j = 0; j < i; ++j) if (rec[j] == tok) { first = false; break; }
        if (!first) continue;
        int count = 0;
        for (int j = i; j < window; ++j) count += rec[j] == tok;
        float l = row[tok];
        if (repeat_penalty != 1.f) l = l > 0.f ? l / repeat_penalty : l * repeat_penalty;
        l -= presence_penalty + frequency_penalty * (float)count;
        row[tok] = l;
    }
}

// With few rows, one block per row leaves most of the GPU idle while it reads 150,000 logits four times over.  For a
// small top-k the row is therefore cut into chunks, grid (chunks, B): this kernel applies the penalties to its chunk and
// leaves the chunk's maximum and adds its counts of tokens by the top 10 bits of their key onto the row's; sample_gather_kernel
// finds the bin of the k-th largest key and gathers the tokens from that bin up; sample_kernel goes on from there.
__global__ void __launch_bounds__(SPLIT_THREADS)
sample_scan_kernel(float* logits, int V, int chunk, const int* __restrict__ recent, int window, float repeat_penalty,
                   float presence_penalty, float frequency_penalty, float* __restrict__ part_best,
                   int* __restrict__ part_best_i, int* row_hist) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int BITS = SPLIT_BITS, BINS = SPLIT_BINS;
    __shared__ int whist[SPLIT_WARPS][BINS];
    __shared__ float red_v[SPLIT_WARPS];
    __shared__ int red_i[SPLIT_WARPS];
    const int c = blockIdx.x, b = blockIdx.y, n_chunks = gridDim.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float* row = logits + (size_t)b * V;
    const int i0 = min(V, c * chunk), i1 = min(V, i0 + chunk);
    if (recent && window > 0 && (repeat_penalty != 1.f || presence_penalty != 0.f || frequency_penalty != 0.f))
        apply_penalties(row, i0, i1, recent + (size_t)b * window, window, repeat_penalty, presence_penalty, frequency_penalty);
    for (int i = tid; i < SPLIT_WARPS * BINS; i += blockDim.x) (&whist[0][0])[i] = 0;
    __syncthreads();
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    int* my_hist = whist[warp];
    for_each_logit(row + i0, i1 - i0, [&](int i, float l, bool valid) {
        if (valid && (l > best || (l == best && i0 + i < best_i))) { best = l; best_i = i0 + i; }
        const unsigned live = __ballot_sync(0xffffffffu, valid);
        if (valid) {
            const int bin = (int)(order_key(l) >> (32 - BITS));
            const unsigned peers = __match_any_sync(live, bin);
            if (lane == __ffs(peers) - 1) my_hist[bin] += __popc(peers);
        }
        __syncwarp();
    });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { red_v[warp] = best; red_i[warp] = best_i; }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < SPLIT_WARPS; ++w)
            if (red_v[w] > best || (red_v[w] == best && red_i[w] < best_i)) { best = red_v[w]; best_i = red_i[w]; }
        part_best[(size_t)b * n_chunks + c] = best;
        part_best_i[(size_t)b * n_chunks + c] = best_i;
    }
    for (int bin = tid; bin < BINS; bin += blockDim.x) {                 // onto the row's counts (integers: any order gives the same)
        int n = 0;
        for (int w = 0; w < SPLIT_WARPS; ++w) n += whist[w][bin];
        if (n) atomicAdd(&row_hist[(size_t)b * BINS + bin], n);
    }
}

__global__ void __launch_bounds__(SPLIT_THREADS)
sample_gather_kernel(const float* __restrict__ logits, int V, int chunk, int top_k, const float* __restrict__ part_best,
                     const int* __restrict__ part_best_i, const int* __restrict__ row_hist, float* __restrict__ best_out,
                     int* __restrict__ best_i_out, int* __restrict__ info, int* count, int* __restrict__ cand_id,
                     float* __restrict__ cand_l, double* __restrict__ part_mass, float inv_temp) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int BITS = SPLIT_BITS, BINS = SPLIT_BINS;
    __shared__ int hist_n[BINS];
    __shared__ int sh_bin, sh_above, sh_at, sh_fits;
    __shared__ float sh_best;
    __shared__ double red_d[SPLIT_WARPS];
    const int c = blockIdx.x, b = blockIdx.y, n_chunks = gridDim.x, tid = threadIdx.x;
    for (int bin = tid; bin < BINS; bin += blockDim.x) hist_n[bin] = row_hist[(size_t)b * BINS + bin];
    __syncthreads();
    if (top_k <= 0) {                                                    // temperature alone: only the masses are wanted
        if (tid == 0) { sh_bin = BINS; sh_above = 0; sh_at = 0; }
    } else if (tid < 32) {
        find_count_bin<BINS / 32>(hist_n, 0, top_k, &sh_bin, &sh_above, &sh_at);   // the k-th largest key's bin
    }
    __syncthreads();
    if (tid == 0) {
        const int bin = sh_bin, run = sh_above;
        sh_fits = run + sh_at <= SAMPLE_CAND_MAX;
        float best = part_best[(size_t)b * n_chunks];
        int best_i = part_best_i[(size_t)b * n_chunks];
        for (int k = 1; k < n_chunks; ++k) {
            const float v = part_best[(size_t)b * n_chunks + k];
            const int vi = part_best_i[(size_t)b * n_chunks + k];
            if (v > best || (v == best && vi < best_i)) { best = v; best_i = vi; }
        }
        sh_best = best;
        if (c == 0) {
            best_out[b] = best;
            best_i_out[b] = best_i;
            info[4 * b] = bin;
            info[4 * b + 1] = run;
            info[4 * b + 2] = sh_fits ? 0 : 1;
            info[4 * b + 3] = BITS;
        }
    }
    __syncthreads();
    if (!sh_fits) return;                                                // the sampling kernel does this row by itself
    const int cut_bin = sh_bin;
    const float* row = logits + (size_t)b * V;
    const int i0 = min(V, c * chunk), i1 = min(V, i0 + chunk);
    const float best = sh_best;
    double mass = 0.0;
    for_each_logit(row + i0, i1 - i0, [&](int i, float l, bool valid) {
        if (valid && (int)(order_key(l) >> (32 - BITS)) >= cut_bin) {
            const int slot = atomicAdd(&count[b], 1);
            if (slot < SAMPLE_CAND_MAX) {
                cand_id[(size_t)b * SAMPLE_CAND_MAX + slot] = i0 + i;
                cand_l[(size_t)b * SAMPLE_CAND_MAX + slot] = l;
            }
        }
        if (part_mass && valid) mass += (double)expf((l - best) * inv_temp);
    });
    if (part_mass) {                                                     // top-p over the whole row wants the whole row's mass
        mass = block_sum(mass, red_d);
        if (tid == 0) part_mass[(size_t)b * n_chunks + c] = mass;
    }
}

// `count` (a power of two) 64-bit words in shared memory into ascending order (a bitonic network); the whole block calls it.
__device__ void sort_words(unsigned long long* w, int count) {
    for (int k = 2; k <= count; k <<= 1)
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = threadIdx.x; i < count; i += blockDim.x) {
                const int other = i ^ j;
                if (other > i) {
                    const bool ascending = (i & k) == 0;
                    const unsigned long long a = w[i], o = w[other];
                    if ((a > o) == ascending) { w[i] = o; w[other] = a; }
                }
            }
            __syncthreads();
        }
}

// logits [B, V] float (changed in place when penalties apply); recent [B, window] token ids
// seen lately, -1 where empty; sequence_index [B] and step (+ *step_add, if given: a counter on
// the device, for steps replayed from a CUDA graph) key the random stream, with the seed (read from *seed_from
// instead, if that is given: a seed on the device, so that a captured graph serves every seed); out_ids [B];
// out_u [B] optional: the uniform numbers that were used.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(float* logits, int V, const int* __restrict__ recent, int window, float repeat_penalty,
              float presence_penalty, float frequency_penalty, float temperature, int top_k, float top_p,
              unsigned long long seed, const unsigned long long* __restrict__ seed_from,
              const int* __restrict__ sequence_index, unsigned int step,
              const unsigned int* __restrict__ step_add, int* __restrict__ out_ids, double* out_u, const Gathered pre) {
    pdl_wait();
    pdl_launch_dependents();
    if (seed_from) seed = *seed_from;
    extern __shared__ __align__(8) unsigned char sample_smem[];      // a histogram per warp: [warps][256] masses, then counts
    double* whist = reinterpret_cast<double*>(sample_smem);
    int* whist_n = reinterpret_cast<int*>(whist + SAMPLE_WARPS * 256);
    __shared__ double hist[256];
    __shared__ int hist_n[256];
    __shared__ double sh_above;
    __shared__ uint32_t sh_prefix;
    __shared__ float red_v[32];
    __shared__ int red_i[32];
    __shared__ double red_d[SAMPLE_THREADS / 32];
    __shared__ int sh_pick;

    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float* row = logits + (size_t)b * V;

    // The split kernels have been over this row (penalties, maximum, the tokens from the cut's bin up gathered)?
    const bool given = pre.count != nullptr && pre.info[4 * b + 2] == 0;
    if (pre.count)
        for (int bin = tid; bin < SPLIT_BINS; bin += blockDim.x) pre.hist[(size_t)b * SPLIT_BINS + bin] = 0;   // for the next launch

    // 1. penalties over the recent tokens, each distinct token once
    if (!pre.count && recent && window > 0 && (repeat_penalty != 1.f || presence_penalty != 0.f || frequency_penalty != 0.f)) {
        apply_penalties(row, 0, V, recent + (size_t)b * window, window, repeat_penalty, presence_penalty, frequency_penalty);
        __syncthreads();
    }

    // 2. maximum, lowest id among equals.  With a small top-k ahead, the same pass counts the tokens by the top byte of
    // their key (a histogram per warp, the lanes that hit a bin counted by one of them).
    const bool small_k = temperature > 0.f && top_k > 0 && top_k < V && top_k <= SAMPLE_THREADS;
    // top-p with no top-k is first tried on the SAMPLE_THREADS most likely tokens: it nearly always ends among them
    const bool p_try = temperature > 0.f && top_p < 1.f && !(top_k > 0 && top_k < V) && V > SAMPLE_THREADS;
    const bool narrow = small_k || p_try;
    const int k_eff = small_k ? top_k : SAMPLE_THREADS;
    int* top_hist = reinterpret_cast<int*>(sample_smem);                 // [warps][256], the first 32 KB
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    if (given) {
        // nothing to read
    } else if (narrow) {
        for (int i = tid; i < SAMPLE_WARPS * 256; i += blockDim.x) top_hist[i] = 0;
        __syncthreads();
        int* my_hist = top_hist + warp * 256;
        for_each_logit(row, V, [&](int i, float l, bool valid) {
            if (valid && (l > best || (l == best && i < best_i))) { best = l; best_i = i; }
            const unsigned live = __ballot_sync(0xffffffffu, valid);
            if (valid) {
                const int bin = (int)(order_key(l) >> 24);
                const unsigned peers = __match_any_sync(live, bin);
                if (lane == __ffs(peers) - 1) my_hist[bin] += __popc(peers);
            }
            __syncwarp();
        });
    } else {
        int scalar_from = 0;
        if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {  // 16-byte loads, four in flight per thread: one block reads a row
            const float4* row4 = reinterpret_cast<const float4*>(row);   // of 150,000 logits in a few microseconds
            const int n4 = V >> 2;
#pragma unroll 4
            for (int i = tid; i < n4; i += blockDim.x) {
                const float4 v = row4[i];
                const float l4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (l4[e] > best || (l4[e] == best && 4 * i + e < best_i)) { best = l4[e]; best_i = 4 * i + e; }
            }
            scalar_from = n4 << 2;
        }
        for (int i = scalar_from + tid; i < V; i += blockDim.x) {
            const float l = row[i];
            if (l > best || (l == best && i < best_i)) { best = l; best_i = i; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { red_v[warp] = best; red_i[warp] = best_i; }
    __syncthreads();
    best = red_v[0]; best_i = red_i[0];
    for (int w = 1; w < (blockDim.x >> 5); ++w)
        if (red_v[w] > best || (red_v[w] == best && red_i[w] < best_i)) { best = red_v[w]; best_i = red_i[w]; }
    if (given) { best = pre.best[b]; best_i = pre.best_i[b]; }
    if (best_i == 0x7fffffff) best_i = 0;            // a row of NaN or -inf: the reference's loop keeps 0
    if (temperature <= 0.f) {
        if (tid == 0) out_ids[b] = best_i;
        return;
    }

    // 3. top-k, 4. top-p
    const float inv_temp = 1.f / temperature;
    Cut cut;
    cut.key = 0u;
    cut.id_limit = V;
    if (!small_k && top_k > 0 && top_k < V)
        cut = radix_cut(row, V, cut, false, (double)top_k, best, inv_temp, whist, whist_n, hist, hist_n, &sh_above, &sh_prefix);

    auto block_mass = [&](const Cut& c) -> double {
        double mine = 0.0;
        for_each_logit(row, V, [&](int i, float l, bool valid) {
            if (valid && kept(c, order_key(l), i)) mine += (double)expf((l - best) * inv_temp);
        });
        return block_sum(mine, red_d);
    };

    if (narrow) {
        // Few tokens will be left (at most one per thread).  The histogram of the first pass says in which bin of the top
        // byte the k-th largest key lies; if that bin and the bins above it hold few tokens, a second pass gathers those into
        // shared memory and everything else (the exact cut, ties, top-p, the draw) happens there.  Otherwise the general
        // selection runs and a pass gathers the kept tokens.  Either way the row is not read again after that.
        constexpr int CAND_MAX = SAMPLE_CAND_MAX;
        float* wide_l = reinterpret_cast<float*>(sample_smem + 32768);    // gathered candidates: the last 64 KB
        int* wide_id = reinterpret_cast<int*>(wide_l + CAND_MAX);
        int* cand_id = reinterpret_cast<int*>(sample_smem);               // the kept tokens, as found: over the histogram
        float* cand_l = reinterpret_cast<float*>(cand_id + SAMPLE_THREADS);
        int* by_id = reinterpret_cast<int*>(cand_l + SAMPLE_THREADS);     // in id order
        float* by_id_l = reinterpret_cast<float*>(by_id + SAMPLE_THREADS);
        double* by_rank_m = reinterpret_cast<double*>(by_id_l + SAMPLE_THREADS);   // masses, largest logit first
        __shared__ int cand_n, keep_n, wide_n, sh_bin, sh_above_n, sh_at_n, sh_limit, sh_beyond;
        __syncthreads();
        if (!given)
            for (int bin = tid; bin < 256; bin += blockDim.x) {           // the warps' counts, added up
                int n = 0;
                for (int w = 0; w < SAMPLE_WARPS; ++w) n += top_hist[w * 256 + bin];
                hist_n[bin] = n;
            }
        if (tid == 0) { cand_n = 0; wide_n = 0; sh_pick = -1; sh_beyond = 0; }
        __syncthreads();
        if (given) {
            if (tid == 0) {
                sh_bin = pre.info[4 * b];
                sh_above_n = pre.info[4 * b + 1];
                sh_at_n = 0;
                wide_n = min(pre.count[b], CAND_MAX);
            }
        } else if (tid < 32) {
            find_count_bin<8>(hist_n, 0, k_eff, &sh_bin, &sh_above_n, &sh_at_n);   // the k-th largest key has this top byte
        }
        __syncthreads();
        const int cut_bin = sh_bin, above_bin = sh_above_n;
        if (above_bin + sh_at_n <= CAND_MAX) {
            if (given) {
                for (int e = tid; e < wide_n; e += blockDim.x) {
                    wide_id[e] = pre.id[(size_t)b * CAND_MAX + e];
                    wide_l[e] = pre.logit[(size_t)b * CAND_MAX + e];
                }
            } else {
                for_each_logit(row, V, [&](int i, float l, bool valid) {
                    if (valid && (int)(order_key(l) >> 24) >= cut_bin) {
                        const int slot = atomicAdd(&wide_n, 1);
                        if (slot < CAND_MAX) { wide_id[slot] = i; wide_l[slot] = l; }
                    }
                });
            }
            __syncthreads();
            const int n_wide = min(wide_n, CAND_MAX);
            if (p_try && given && pre.mass) {
                // top-p alone: if even all the gathered tokens do not reach the share, the general way has to do it
                double all = 0.0, got = 0.0;
                for (int c = 0; c < pre.n_chunks; ++c) all += pre.mass[(size_t)b * pre.n_chunks + c];
                for (int e = tid; e < n_wide; e += blockDim.x) got += (double)expf((wide_l[e] - best) * inv_temp);
                got = block_sum(got, red_d);
                if (tid == 0 && got < (double)top_p * all * (1.0 - 1e-9)) sh_beyond = 1;
                __syncthreads();
            }
            if (!sh_beyond) {
            // the exact cut among the tokens of the cut bin: the rest of the key, up to 8 bits at a time, on the gathered tokens
            int low = given ? 32 - SPLIT_BITS : 24;                       // bits of the key not yet decided
            uint32_t prefix = (uint32_t)cut_bin << low, mask = ~0u << low;
            int above = above_bin;
            while (low > 0) {
                const int width = min(8, low), shift = low - width;
                const uint32_t field = (1u << width) - 1u;
                for (int bin = tid; bin < 256; bin += blockDim.x) hist_n[bin] = 0;
                __syncthreads();
                for (int e = tid; e < n_wide; e += blockDim.x) {
                    const uint32_t key = order_key(wide_l[e]);
                    if ((key & mask) == prefix) atomicAdd(&hist_n[(key >> shift) & field], 1);
                }
                __syncthreads();
                if (tid < 32) find_count_bin<8>(hist_n, above, k_eff, &sh_bin, &sh_above_n, &sh_at_n);
                __syncthreads();
                prefix |= (uint32_t)sh_bin << shift;
                mask |= field << shift;
                above = sh_above_n;
                low = shift;
                __syncthreads();
            }
            const int n_at = sh_at_n, needed = max(1, k_eff - above);   // tokens with exactly the cut key, and how many are kept
            if (tid == 0) sh_limit = V;
            __syncthreads();
            if (needed < n_at) {                                          // a tie across the cut: the lowest ids
                for (int e = tid; e < n_wide; e += blockDim.x) {
                    if (order_key(wide_l[e]) != prefix) continue;
                    int rank = 0;
                    for (int j = 0; j < n_wide; ++j) rank += order_key(wide_l[j]) == prefix && wide_id[j] < wide_id[e];
                    if (rank == needed - 1) sh_limit = wide_id[e];
                }
            }
            __syncthreads();
            cut.key = prefix;
            cut.id_limit = sh_limit;
            for (int e = tid; e < n_wide; e += blockDim.x) {
                if (kept(cut, order_key(wide_l[e]), wide_id[e])) {
                    const int slot = atomicAdd(&cand_n, 1);
                    if (slot < SAMPLE_THREADS) { cand_id[slot] = wide_id[e]; cand_l[slot] = wide_l[e]; }
                }
            }
            }
        } else if (small_k) {
            cut = radix_cut(row, V, cut, false, (double)top_k, best, inv_temp, whist, whist_n, hist, hist_n, &sh_above, &sh_prefix);
            for_each_logit(row, V, [&](int i, float l, bool valid) {
                if (valid && kept(cut, order_key(l), i)) {
                    const int slot = atomicAdd(&cand_n, 1);
                    if (slot < SAMPLE_THREADS) { cand_id[slot] = i; cand_l[slot] = l; }
                }
            });
        } else if (tid == 0) {
            sh_beyond = 1;                                               // too many tokens share the top byte: the general way
        }
        __syncthreads();
        const int n = min(cand_n, SAMPLE_THREADS);
        int padded = 1;
        while (padded < n) padded <<= 1;
        unsigned long long* words = reinterpret_cast<unsigned long long*>(wide_l);   // (the gathered tokens are done with)
        const bool few = n <= 128;      // few tokens: each counts those before it; many: a sorting network (a barrier per stage)
        if (few) {
            if (tid < n) {                                               // into id order
                const int id = cand_id[tid];
                int pos = 0;
                for (int j = 0; j < n; ++j) pos += cand_id[j] < id;
                by_id[pos] = id;
                by_id_l[pos] = cand_l[tid];
            }
        } else {
            for (int i = tid; i < padded; i += blockDim.x)
                words[i] = i < n ? ((unsigned long long)(uint32_t)cand_id[i] << 32) | __float_as_uint(cand_l[i]) : ~0ull;
            __syncthreads();
            sort_words(words, padded);
            if (tid < n) {
                by_id[tid] = (int)(words[tid] >> 32);
                by_id_l[tid] = __uint_as_float((uint32_t)words[tid]);
            }
        }
        __syncthreads();
        const bool have = tid < n;
        const int id = have ? by_id[tid] : 0;
        const float l = have ? by_id_l[tid] : 0.f;
        const double m = have ? (double)expf((l - best) * inv_temp) : 0.0;
        bool keep = have;
        if (top_p < 1.f && !sh_beyond) {
            double total = block_sum(m, red_d);
            if (p_try) {                                                 // the share is of the whole row's mass
                Cut all;
                all.key = 0u;
                all.id_limit = V;
                if (given && pre.mass) {
                    total = 0.0;
                    for (int c = 0; c < pre.n_chunks; ++c) total += pre.mass[(size_t)b * pre.n_chunks + c];
                } else {
                    total = block_mass(all);
                }
            }
            // rank: larger logits first, lower ids (= earlier places in id order) first among equals
            if (few) {
                if (have) {
                    int rank = 0;
                    for (int j = 0; j < n; ++j) rank += by_id_l[j] > l || (by_id_l[j] == l && j < tid);
                    by_rank_m[rank] = m;
                    cand_id[tid] = rank;                                 // (the gather's arrays are free again)
                }
            } else {
                for (int i = tid; i < padded; i += blockDim.x)
                    words[i] = i < n ? ((unsigned long long)(uint32_t)~order_key(by_id_l[i]) << 32) | (unsigned)i : ~0ull;
                __syncthreads();
                sort_words(words, padded);
                if (have) {
                    const int place = (int)(uint32_t)words[tid];         // the token of rank tid
                    by_rank_m[tid] = (double)expf((by_id_l[place] - best) * inv_temp);
                    cand_id[place] = tid;
                }
            }
            if (tid == 0) keep_n = n + 1;
            __syncthreads();
            {                                                            // the smallest prefix whose share reaches top_p:
                const double target = (double)top_p * total;             // a scan over the masses in rank order
                const double mr = tid < n ? by_rank_m[tid] : 0.0;
                double incl = mr;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const double up = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += up;
                }
                if (lane == 31) red_d[warp] = incl;
                __syncthreads();
                for (int w = 0; w < warp; ++w) incl += red_d[w];
                if (tid < n && incl >= target) atomicMin(&keep_n, tid + 1);
                __syncthreads();
                if (tid == 0) {
                    if (keep_n > n) {                                    // never reached
                        if (p_try) sh_beyond = 1;                        // the prefix ends beyond these tokens: the general way
                        keep_n = n;                                      // (else: rounding left the total short; keep all)
                    }
                    if (keep_n < 1) keep_n = 1;
                }
            }
            __syncthreads();
            keep = have && cand_id[tid] < keep_n;
        }
        if (!sh_beyond) {
            // the draw: a scan over the kept tokens in id order
            const double mine = keep ? m : 0.0;
            double incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const double up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            __syncthreads();
            if (lane == 31) red_d[warp] = incl;
            __syncthreads();
            double before = 0.0, total = 0.0;
            for (int w = 0; w < (blockDim.x >> 5); ++w) {
                if (w < warp) before += red_d[w];
                total += red_d[w];
            }
            before += incl - mine;
            const double u = philox_uniform(seed, (unsigned int)(sequence_index ? sequence_index[b] : b),
                                            step + (step_add ? *step_add : 0u));
            const double r = u * total;
            if (mine > 0.0 && r > before && r <= before + mine) sh_pick = id;
            __syncthreads();
            if (tid == 0) {
                out_ids[b] = sh_pick >= 0 ? sh_pick : best_i;
                if (out_u) out_u[b] = u;
                if (pre.count) pre.count[b] = 0;                         // as the next launch expects it
            }
            return;
        }
        // top-p alone, and its tokens are more than were looked at: start again with every token
        __syncthreads();
        if (tid == 0 && pre.count) pre.count[b] = 0;
        cut.key = 0u;
        cut.id_limit = V;
    }

    if (top_p < 1.f) {
        const double total = block_mass(cut);
        cut = radix_cut(row, V, cut, true, (double)top_p * total, best, inv_temp, whist, whist_n, hist, hist_n, &sh_above, &sh_prefix);
    }

    // 5. one draw, walking the kept tokens in id order.  Every warp owns a run of ids (a multiple of 128, so that its
    // lanes read 16 bytes each, 4 ids in a row): first each warp adds up its run, then the one warp whose run holds the
    // drawn point walks it again, 128 ids at a time with a scan over its lanes.
    const double u = philox_uniform(seed, (unsigned int)(sequence_index ? sequence_index[b] : b),
                                    step + (step_add ? *step_add : 0u));
    // Temperature alone after the split kernels: the chunks' masses say which chunk holds the drawn point; only that
    // chunk is walked.
    int lo = 0, hi = V;
    double base = 0.0, all = -1.0;
    if (given && pre.mass && !narrow) {
        const double* mass = pre.mass + (size_t)b * pre.n_chunks;
        all = 0.0;
        for (int c = 0; c < pre.n_chunks; ++c) all += mass[c];
        const double r0 = u * all;
        int chosen = -1, last = 0;
        double run = 0.0, last_base = 0.0;
        for (int c = 0; c < pre.n_chunks; ++c) {
            const double m = mass[c];
            if (m > 0.0) {
                last = c;
                last_base = run;
                if (chosen < 0 && r0 <= run + m) { chosen = c; base = run; }
            }
            run += m;
        }
        if (chosen < 0) { chosen = last; base = last_base; }            // rounding at the very end
        lo = min(V, chosen * pre.chunk);
        hi = min(V, lo + pre.chunk);
    }
    const int n_warps = (int)(blockDim.x >> 5);
    const int per_warp = ((hi - lo + n_warps - 1) / n_warps + 127) / 128 * 128;
    const int w0 = min(hi, lo + warp * per_warp), w1 = min(hi, w0 + per_warp);
    const bool vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
    auto masses = [&](int i0, double* m) -> double {          // masses of the 4 ids from i0 on (0 where not kept), and their sum
        float l4[4] = {0.f, 0.f, 0.f, 0.f};
        if (vec && i0 + 3 < V) {
            const float4 v = *reinterpret_cast<const float4*>(row + i0);
            l4[0] = v.x; l4[1] = v.y; l4[2] = v.z; l4[3] = v.w;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) if (i0 + e < V) l4[e] = row[i0 + e];
        }
        double sum = 0.0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = i0 + e;
            m[e] = (i < w1 && kept(cut, order_key(l4[e]), i)) ? (double)expf((l4[e] - best) * inv_temp) : 0.0;
            sum += m[e];
        }
        return sum;
    };
    double mine = 0.0;
    for (int c0 = w0; c0 < w1; c0 += 128) {
        double m[4];
        mine += masses(c0 + 4 * lane, m);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    if (lane == 0) red_d[warp] = mine;
    if (tid == 0) sh_pick = -1;
    __syncthreads();
    double before_warp = base, total = 0.0;
    for (int w = 0; w < n_warps; ++w) {
        if (w < warp) before_warp += red_d[w];
        total += red_d[w];
    }
    if (all >= 0.0) total = all;
    const double r = u * total;
    if (red_d[warp] > 0.0 && r > before_warp && r <= before_warp + red_d[warp]) {    // this warp's run holds the point
        double running = before_warp;
        int pick = -1;
        for (int c0 = w0; c0 < w1 && pick < 0; c0 += 128) {
            const int i0 = c0 + 4 * lane;
            double m[4];
            const double sum = masses(i0, m);
            double incl = sum;                           // inclusive scan over the lanes
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const double up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            const double before = running + incl - sum;
            int found = -1;
            if (sum > 0.0 && r > before && r <= before + sum) {
                double run = before;
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (m[e] > 0.0 && (found < 0 || run < r)) { run += m[e]; found = i0 + e; }
            }
            // at most one lane finds it; rounding at a chunk's edge may leave it to the next chunk or to the fallback
            const unsigned who = __ballot_sync(0xffffffffu, found >= 0);
            if (who) pick = __shfl_sync(0xffffffffu, found, __ffs(who) - 1);
            running += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) sh_pick = pick;
    }
    __syncthreads();
    if (tid == 0) {
        out_ids[b] = sh_pick >= 0 ? sh_pick : best_i;     // rounding at the very end of the walk: the mode
        if (pre.count) pre.count[b] = 0;
        if (out_u) out_u[b] = u;
    }
}

// Greedy with few rows: the row cut into chunks as above, grid (chunks, B): penalties and the maximum of the chunk (lowest
// id among equals); then one warp per row picks among the chunks.  8 rows of 151,936 logits: 6 us against 10-13 with one
// block per row, which reads its 600 KB alone.
__global__ void __launch_bounds__(SPLIT_THREADS)
sample_argmax_chunk_kernel(float* logits, int V, int chunk, const int* __restrict__ recent, int window, float repeat_penalty,
                           float presence_penalty, float frequency_penalty, float* __restrict__ part_best,
                           int* __restrict__ part_best_i) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float red_v[SPLIT_WARPS];
    __shared__ int red_i[SPLIT_WARPS];
    const int c = blockIdx.x, b = blockIdx.y, n_chunks = gridDim.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float* row = logits + (size_t)b * V;
    const int i0 = min(V, c * chunk), i1 = min(V, i0 + chunk);
    if (recent && window > 0 && (repeat_penalty != 1.f || presence_penalty != 0.f || frequency_penalty != 0.f)) {
        apply_penalties(row, i0, i1, recent + (size_t)b * window, window, repeat_penalty, presence_penalty, frequency_penalty);
        __syncthreads();
    }
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for_each_logit(row + i0, i1 - i0, [&](int i, float l, bool valid) {
        if (valid && (l > best || (l == best && i0 + i < best_i))) { best = l; best_i = i0 + i; }
    });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { red_v[warp] = best; red_i[warp] = best_i; }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < SPLIT_WARPS; ++w)
            if (red_v[w] > best || (red_v[w] == best && red_i[w] < best_i)) { best = red_v[w]; best_i = red_i[w]; }
        part_best[(size_t)b * n_chunks + c] = best;
        part_best_i[(size_t)b * n_chunks + c] = best_i;
    }
}

__global__ void __launch_bounds__(32)
sample_argmax_pick_kernel(const float* __restrict__ part_best, const int* __restrict__ part_best_i, int n_chunks,
                          int* __restrict__ out_ids) {
    pdl_wait();
    pdl_launch_dependents();
    const int b = blockIdx.x, lane = threadIdx.x;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int c = lane; c < n_chunks; c += 32) {
        const float v = part_best[(size_t)b * n_chunks + c];
        const int i = part_best_i[(size_t)b * n_chunks + c];
        if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) out_ids[b] = best_i == 0x7fffffff ? 0 : best_i;     // a row of NaN or -inf: the reference's loop keeps 0
}

// Chunks a row for greedy sampling (0: one block does the whole row).
static int greedy_chunks(int B, int V) {
    int dev = 0, n_sm = 148;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) n_sm = 148;
    int chunks = 4 * n_sm / B;
    if (chunks > 32) chunks = 32;
    if (chunks > V / 2048) chunks = V / 2048;
    return chunks < 16 ? 0 : chunks;          // as for the other split kernels: with more than 37 rows a block per row is as fast
}

// How the row is cut for the split kernels: 0 chunks = one block does the whole row.
static int split_chunks(int B, int V, float temperature, int top_k, float top_p) {
    const bool small_k = top_k > 0 && top_k < V && top_k <= SAMPLE_THREADS;
    const bool p_try = top_p < 1.f && !(top_k > 0 && top_k < V) && V > SAMPLE_THREADS;      // as in sample_kernel
    const bool t_only = !(top_p < 1.f) && !(top_k > 0 && top_k < V);                         // temperature alone
    if (!(temperature > 0.f) || !(small_k || p_try || t_only)) return 0;
    static int n_sm = 0;
    if (!n_sm) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) n_sm = 148;
    }
    int chunks = 4 * n_sm / B;                                       // four blocks of 256 threads find room on an SM
    if (chunks > 32) chunks = 32;
    if (chunks > V / 2048) chunks = V / 2048;
    // With fewer than 16 chunks a row (more than 37 rows on 148 SMs, or a small vocabulary) the three kernels cost more
    // than they save: measured 87 against 64 us at 64 rows of 151,936 logits, 41 against 63 us at 16 rows.  Not so for
    // top-p alone: a block on its own counts by the key's top byte only, too coarse to gather 1,024 tokens of a wide
    // distribution, and then takes the general way (135 against 505 us at 64 rows).
    return chunks < (p_try ? 2 : 16) ? 0 : chunks;
}

// Bytes of scratch that qwb_sample wants for these arguments (0: none); 16-byte aligned memory, any contents.
extern "C" int qwb_sample_scratch_bytes(int B, int V, float temperature, int top_k, float top_p) {
    if (!(temperature > 0.f)) return greedy_chunks(B, V) ? B * 32 * 8 : 0;
    const int chunks = split_chunks(B, V, temperature, top_k, top_p);     // at most 32 chunks of at most 296 rows: 20 MB
    if (!chunks) return 0;
    return B * chunks * (2 + 2) * 4 + B * (2 + 4) * 4 + B * SAMPLE_CAND_MAX * 8;
}

// scratch: qwb_sample_scratch_bytes() bytes, or null (then a block does a whole row whatever the arguments);
// counters: [B][1 + 1024] int, zero before the first call (the kernels leave them zero), needed with scratch.
extern "C" int qwb_sample(float* logits, int B, int V, const int* recent, int window, float repeat_penalty,
                          float presence_penalty, float frequency_penalty, float temperature, int top_k, float top_p,
                          unsigned long long seed, const unsigned long long* seed_from, const int* sequence_index,
                          unsigned int step, const unsigned int* step_add, int* out_ids, double* out_u, void* scratch,
                          int* counters, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (V <= 0) return qwb_fail(QWB_ERR_ARG, "sample: bad vocabulary size %d", V);
    if (temperature > 0.f && !(top_p > 0.f)) return qwb_fail(QWB_ERR_ARG, "sample: top_p must be > 0, got %g", (double)top_p);
    if (repeat_penalty <= 0.f) return qwb_fail(QWB_ERR_ARG, "sample: repeat_penalty must be > 0, got %g", (double)repeat_penalty);
    const size_t smem = (size_t)SAMPLE_WARPS * 256 * (sizeof(double) + sizeof(int));
    static bool sized = false;
    if (!sized) {
        cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "sample: %s", cudaGetErrorString(e));
        sized = true;
    }
    if (!(temperature > 0.f) && scratch && greedy_chunks(B, V)) {
        if ((uintptr_t)scratch % 16) return qwb_fail(QWB_ERR_ARG, "sample: the scratch memory must be 16-byte aligned");
        const int chunks = greedy_chunks(B, V);
        float* part_best = reinterpret_cast<float*>(scratch);
        int* part_best_i = reinterpret_cast<int*>(part_best + (size_t)B * chunks);
        const int chunk = ((V + chunks - 1) / chunks + 3) / 4 * 4;
        qwb_launch(sample_argmax_chunk_kernel, dim3(chunks, B), SPLIT_THREADS, 0, stream, logits, V, chunk, recent, window,
                   repeat_penalty, presence_penalty, frequency_penalty, part_best, part_best_i);
        qwb_launch(sample_argmax_pick_kernel, B, 32, 0, stream, (const float*)part_best, (const int*)part_best_i, chunks, out_ids);
        return qwb_check_launch("sample");
    }
    Gathered pre = {};
    const int chunks = scratch && counters ? split_chunks(B, V, temperature, top_k, top_p) : 0;
    if (chunks) {
        if ((uintptr_t)scratch % 16) return qwb_fail(QWB_ERR_ARG, "sample: the scratch memory must be 16-byte aligned");
        const bool small_k = top_k > 0 && top_k < V && top_k <= SAMPLE_THREADS;
        const bool p_try = top_p < 1.f && !(top_k > 0 && top_k < V) && V > SAMPLE_THREADS;
        double* part_mass = reinterpret_cast<double*>(scratch);
        float* part_best = reinterpret_cast<float*>(part_mass + (size_t)B * chunks);
        int* row_hist = counters + B;
        int* part_best_i = reinterpret_cast<int*>(part_best + (size_t)B * chunks);
        float* best = reinterpret_cast<float*>(part_best_i + (size_t)B * chunks);
        int* best_i = reinterpret_cast<int*>(best + B);
        int* info = best_i + B;
        int* cand_id = info + 4 * (size_t)B;
        float* cand_l = reinterpret_cast<float*>(cand_id + (size_t)B * SAMPLE_CAND_MAX);
        const int chunk = ((V + chunks - 1) / chunks + 3) / 4 * 4;       // a multiple of 4: 16-byte loads stay possible
        qwb_launch(sample_scan_kernel, dim3(chunks, B), SPLIT_THREADS, 0, stream, logits, V, chunk, recent, window, repeat_penalty,
                   presence_penalty, frequency_penalty, part_best, part_best_i, row_hist);
        qwb_launch(sample_gather_kernel, dim3(chunks, B), SPLIT_THREADS, 0, stream, (const float*)logits, V, chunk,
                   small_k ? top_k : (p_try ? SAMPLE_THREADS : 0), (const float*)part_best, (const int*)part_best_i, (const int*)row_hist, best,
                   best_i, info, counters, cand_id, cand_l, small_k ? (double*)nullptr : part_mass, 1.f / temperature);
        pre.best = best;
        pre.best_i = best_i;
        pre.info = info;
        pre.count = counters;
        pre.hist = row_hist;
        pre.id = cand_id;
        pre.logit = cand_l;
        pre.mass = small_k ? nullptr : part_mass;
        pre.n_chunks = chunks;
        pre.chunk = chunk;
    }
    qwb_launch(sample_kernel, B, SAMPLE_THREADS, smem, stream, logits, V, recent, window, repeat_penalty, presence_penalty,
                                                   frequency_penalty, temperature, top_k, top_p, seed, seed_from,
                                                   sequence_index, step, step_add, out_ids, out_u, pre);
    return qwb_check_launch("sample");
}
