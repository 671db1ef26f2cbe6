// Sampling on the device, one block per sequence, in the reference's order
// (core/sampler.cpp:38-109): penalties over the recent tokens; greedy if the temperature
// is <= 0 (the lowest id wins a tie); else top-k by logit, softmax with temperature,
// top-p (the smallest descending prefix whose share reaches top_p), and one draw.
//
// Nothing is sorted.  The k-th largest logit and the top-p cut are found by radix
// selection over an order-preserving 32-bit key of the logit (four passes of 8 bits
// with a histogram of counts or of probability mass in shared memory); ties at a cut
// are broken toward the lower token id.  The draw walks the kept tokens in id order with
// a uniform number from a counter-based generator (Philox 4x32-10) keyed by the seed,
// the sequence's own index and the step, so a sequence's tokens do not depend on what
// else is in the batch.
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

// Radix selection.  Among the tokens kept by `within`, finds the cut such that the kept
// tokens above it, plus as many tokens at it as needed (lowest ids first), reach `target`:
// a count (by_mass = false) or a probability mass (by_mass = true; mass of token i is
// exp((l_i - lmax) / temperature)).
__device__ Cut radix_cut(const float* row, int V, const Cut within, bool by_mass, double target,
                         float lmax, float inv_temp, double* hist, int* hist_n, double* sh_above, uint32_t* sh_prefix) {
    const int tid = threadIdx.x;
    uint32_t prefix = 0, mask = 0;
    double above = 0.0;
    int n_at = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = tid; i < 256; i += blockDim.x) { hist[i] = 0.0; hist_n[i] = 0; }
        __syncthreads();
        for (int i = tid; i < V; i += blockDim.x) {
            const float l = row[i];
            const uint32_t key = order_key(l);
            if ((key & mask) == prefix && kept(within, key, i)) {
                const int bin = (key >> shift) & 255;
                atomicAdd(&hist[bin], by_mass ? (double)expf((l - lmax) * inv_temp) : 1.0);
                atomicAdd(&hist_n[bin], 1);
            }
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

// logits [B, V] float (changed in place when penalties apply); recent [B, window] token ids
// seen lately, -1 where empty; sequence_index [B] and step (+ *step_add, if given: a counter on
// the device, for steps replayed from a CUDA graph) key the random stream; out_ids [B];
// out_u [B] optional: the uniform numbers that were used.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(float* logits, int V, const int* __restrict__ recent, int window, float repeat_penalty,
              float presence_penalty, float frequency_penalty, float temperature, int top_k, float top_p,
              unsigned long long seed, const int* __restrict__ sequence_index, unsigned int step,
              const unsigned int* __restrict__ step_add, int* __restrict__ out_ids, double* out_u) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ double hist[256];
    __shared__ int hist_n[256];
    __shared__ double sh_above;
    __shared__ uint32_t sh_prefix;
    __shared__ float red_v[32];
    __shared__ int red_i[32];
    __shared__ double red_d[SAMPLE_THREADS / 32];
    __shared__ double warp_base[SAMPLE_THREADS / 32];
    __shared__ int sh_pick;

    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float* row = logits + (size_t)b * V;

    // 1. penalties over the recent tokens, each distinct token once
    if (recent && window > 0 && (repeat_penalty != 1.f || presence_penalty != 0.f || frequency_penalty != 0.f)) {
        const int* rec = recent + (size_t)b * window;
        for (int i = tid; i < window; i += blockDim.x) {
            const int tok = rec[i];
            if (tok < 0 || tok >= V) continue;
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
        __syncthreads();
    }

    // 2. maximum, lowest id among equals
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    int scalar_from = 0;
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {  // 16-byte loads, four in flight per thread: one block reads a row of
        const float4* row4 = reinterpret_cast<const float4*>(row);   // 150,000 logits in a few microseconds
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
    if (top_k > 0 && top_k < V)
        cut = radix_cut(row, V, cut, false, (double)top_k, best, inv_temp, hist, hist_n, &sh_above, &sh_prefix);

    auto block_mass = [&](const Cut& c) -> double {
        double s = 0.0;
        for (int i = tid; i < V; i += blockDim.x) {
            const float l = row[i];
            if (kept(c, order_key(l), i)) s += (double)expf((l - best) * inv_temp);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        __syncthreads();
        if (lane == 0) red_d[warp] = s;
        __syncthreads();
        double total = 0.0;
        for (int w = 0; w < (blockDim.x >> 5); ++w) total += red_d[w];
        return total;
    };

    if (top_p < 1.f) {
        const double total = block_mass(cut);
        cut = radix_cut(row, V, cut, true, (double)top_p * total, best, inv_temp, hist, hist_n, &sh_above, &sh_prefix);
    }

    // 5. one draw, walking the kept tokens in id order; each thread owns a run of ids
    const int seg = (V + blockDim.x - 1) / blockDim.x;
    const int i0 = min(V, tid * seg), i1 = min(V, i0 + seg);
    double mine = 0.0;
    for (int i = i0; i < i1; ++i) {
        const float l = row[i];
        if (kept(cut, order_key(l), i)) mine += (double)expf((l - best) * inv_temp);
    }
    double incl = mine;                                  // inclusive scan inside the warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    if (lane == 31) red_d[warp] = incl;
    if (tid == 0) sh_pick = -1;
    __syncthreads();
    if (tid == 0) {
        double run = 0.0;
        for (int w = 0; w < (blockDim.x >> 5); ++w) { warp_base[w] = run; run += red_d[w]; }
        sh_above = run;                                   // the kept tokens' whole mass
    }
    __syncthreads();
    const double total = sh_above;
    const double u = philox_uniform(seed, (unsigned int)(sequence_index ? sequence_index[b] : b),
                                    step + (step_add ? *step_add : 0u));
    const double r = u * total;
    const double before = warp_base[warp] + incl - mine;
    if (mine > 0.0 && r > before && r <= before + mine) {
        double run = before;
        int pick = -1;
        for (int i = i0; i < i1; ++i) {
            const float l = row[i];
            if (kept(cut, order_key(l), i)) {
                run += (double)expf((l - best) * inv_temp);
                pick = i;
                if (run >= r) break;
            }
        }
        sh_pick = pick;
    }
    __syncthreads();
    if (tid == 0) {
        out_ids[b] = sh_pick >= 0 ? sh_pick : best_i;     // rounding at the very end of the walk: the mode
        if (out_u) out_u[b] = u;
    }
}

extern "C" int qwb_sample(float* logits, int B, int V, const int* recent, int window, float repeat_penalty,
                          float presence_penalty, float frequency_penalty, float temperature, int top_k, float top_p,
                          unsigned long long seed, const int* sequence_index, unsigned int step,
                          const unsigned int* step_add, int* out_ids, double* out_u, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (V <= 0) return qwb_fail(QWB_ERR_ARG, "sample: bad vocabulary size %d", V);
    if (temperature > 0.f && !(top_p > 0.f)) return qwb_fail(QWB_ERR_ARG, "sample: top_p must be > 0, got %g", (double)top_p);
    if (repeat_penalty <= 0.f) return qwb_fail(QWB_ERR_ARG, "sample: repeat_penalty must be > 0, got %g", (double)repeat_penalty);
    qwb_launch(sample_kernel, B, SAMPLE_THREADS, 0, stream, logits, V, recent, window, repeat_penalty, presence_penalty,
                                                   frequency_penalty, temperature, top_k, top_p, seed, sequence_index,
                                                   step, step_add, out_ids, out_u);
    return qwb_check_launch("sample");
}
