// Generation-step kernels: n-gram repeat blocking, top-k / nucleus sampling and the beam-search
// candidate selection. All three are latency-bound single-pass-per-row kernels over a
// [batch, vocab] fp32 matrix that is L2 resident right after the softmax that produced it.
//
// Selection uses an MSB-first radix select over the IEEE bit patterns of the
// (non-negative) probabilities: four passes of 8 bits with per-warp shared-memory histograms of
// (count, mass). This finds the exact k-th largest value and the exact nucleus boundary without
// sorting the vocabulary.
#include <cfloat>

#include "common.cuh"
#include "generation.h"

namespace fs2 {

namespace {

// ------------------------------------------------------------------ n-gram repeat block
__global__ void ngram_repeat_block_kernel(const long long* __restrict__ seqs, float* __restrict__ probs, int S, int V,
                                          int n, float ban_value) {
    const int row = blockIdx.x;
    const long long* s = seqs + static_cast<size_t>(row) * S;
    float* p = probs + static_cast<size_t>(row) * V;
    const int num_starts = S - n + 1;  // windows [i, i + n)
    for (int i = threadIdx.x; i < num_starts; i += blockDim.x) {
        bool match = true;
        for (int j = 0; j < n - 1; ++j) {
            if (s[i + j] != s[S - (n - 1) + j]) {
                match = false;
                break;
            }
        }
        if (match) {
            const long long tok = s[i + n - 1];
            if (tok >= 0 && tok < V) p[tok] = ban_value;
        }
    }
}

// ----------------------------------------------------------------------- radix select
constexpr int SEL_THREADS = 1024;
constexpr int SEL_WARPS = SEL_THREADS / 32;
constexpr int BINS = 256;

struct SelSmem {
    unsigned int cnt[SEL_WARPS][BINS];
    float mass[SEL_WARPS][BINS];
    unsigned int tot_cnt[BINS];
    float tot_mass[BINS];
    float red[32];
    unsigned int prefix;   // bits resolved so far
    float above_mass;      // mass of entries strictly above the resolved prefix range
    unsigned int above_cnt;
    int found;
};

__device__ __forceinline__ unsigned int fbits(float x) { return __float_as_uint(fmaxf(x, 0.f)); }

// Finds the largest bit pattern t such that the set {x : bits(x) >= t} satisfies
//   by_mass: mass{x : bits(x) > t} <= p   (nucleus boundary), or
//   else   : count{x : bits(x) >= t} >= k (k-th largest).
// Returns 0 (keep everything) if the boundary is never crossed.
__device__ unsigned int radix_select(const float* __restrict__ x, int V, bool by_mass, float p, unsigned int k,
                                     SelSmem& sm) {
    const int tid = threadIdx.x, warp = tid >> 5;
    if (tid == 0) {
        sm.prefix = 0;
        sm.above_mass = 0.f;
        sm.above_cnt = 0;
    }
    __syncthreads();
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = tid; i < SEL_WARPS * BINS; i += SEL_THREADS) {
            (&sm.cnt[0][0])[i] = 0;
            (&sm.mass[0][0])[i] = 0.f;
        }
        __syncthreads();
        const unsigned int prefix = sm.prefix;
        const unsigned int hi_mask = (shift == 24) ? 0u : (0xffffffffu << (shift + 8));
        for (int i = tid; i < V; i += SEL_THREADS) {
            const float v = x[i];
            const unsigned int b = fbits(v);
            if ((b & hi_mask) == (prefix & hi_mask)) {
                const unsigned int bin = (b >> shift) & 0xffu;
                atomicAdd(&sm.cnt[warp][bin], 1u);
                if (by_mass) atomicAdd(&sm.mass[warp][bin], fmaxf(v, 0.f));
            }
        }
        __syncthreads();
        if (tid < BINS) {
            unsigned int c = 0;
            float m = 0.f;
            for (int w = 0; w < SEL_WARPS; ++w) {   // fixed order: deterministic totals
                c += sm.cnt[w][tid];
                m += sm.mass[w][tid];
            }
            sm.tot_cnt[tid] = c;
            sm.tot_mass[tid] = m;
        }
        __syncthreads();
        if (tid == 0) {
            float am = sm.above_mass;
            unsigned int ac = sm.above_cnt;
            int found = -1;
            for (int b = BINS - 1; b >= 0; --b) {
                const unsigned int c = sm.tot_cnt[b];
                if (c == 0) continue;
                const bool cross = by_mass ? (am + sm.tot_mass[b] > p) : (ac + c >= k);
                if (cross) {
                    found = b;
                    break;
                }
                am += sm.tot_mass[b];
                ac += c;
            }
            sm.found = found;
            if (found >= 0) {
                sm.prefix = prefix | (static_cast<unsigned int>(found) << shift);
                sm.above_mass = am;
                sm.above_cnt = ac;
            }
        }
        __syncthreads();
        const int found = sm.found;
        __syncthreads();   // nobody may overwrite `found`/`prefix` before every thread has read them
        if (found < 0) return 0u;
    }
    const unsigned int result = sm.prefix;
    __syncthreads();
    return result;
}

__global__ void __launch_bounds__(SEL_THREADS, 1)
sample_kernel(const float* __restrict__ probs, const float* __restrict__ uniform, long long* __restrict__ out, int V,
              float p, int k) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    SelSmem& sm = *reinterpret_cast<SelSmem*>(smem_raw);
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = probs + static_cast<size_t>(row) * V;

    unsigned int thr = 0;
    if (k > 0 && k < V) thr = radix_select(x, V, false, 0.f, static_cast<unsigned int>(k), sm);
    if (p < 1.0f) {
        const unsigned int tp = radix_select(x, V, true, p, 0u, sm);
        thr = tp > thr ? tp : thr;
    }

    // CDF walk over the kept entries in index order: thread t owns the contiguous chunk [t*C, (t+1)*C).
    const int C = (V + SEL_THREADS - 1) / SEL_THREADS;
    const int lo = min(tid * C, V), hi = min(lo + C, V);
    float part = 0.f;
    for (int i = lo; i < hi; ++i) {
        const float v = x[i];
        if (fbits(v) >= thr && v > 0.f) part += v;
    }
    // block-wide exclusive scan of `part`
    float incl = part;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
    }
    __syncthreads();
    if (lane == 31) sm.red[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        float w = (lane < SEL_WARPS) ? sm.red[lane] : 0.f;
        float wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float n = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += n;
        }
        sm.red[lane] = wi - w;                   // exclusive warp offsets
        if (lane == 31) sm.above_mass = wi;      // total kept mass
    }
    if (tid == 0) sm.found = -1;
    __syncthreads();
    const float total = sm.above_mass;
    const float excl = sm.red[warp] + incl - part;
    const float target = fminf(uniform[row], 0.99999994f) * total;
    if (part > 0.f && target >= excl && target < excl + part) {
        float acc = excl;
        int pick = -1;
        for (int i = lo; i < hi; ++i) {
            const float v = x[i];
            if (fbits(v) >= thr && v > 0.f) {
                pick = i;
                acc += v;
                if (acc > target) break;
            }
        }
        sm.found = pick;   // the half-open ranges are disjoint: at most one writer
    }
    __syncthreads();
    if (sm.found < 0) {
        // rounding left the target outside every range (or the row is all zero): take the last kept entry
        int last = -1;
        for (int i = lo; i < hi; ++i) {
            const float v = x[i];
            if (fbits(v) >= thr && v > 0.f) last = i;
        }
        __syncthreads();
        if (last >= 0) atomicMax(&sm.found, last);
        __syncthreads();
    }
    if (tid == 0) out[row] = sm.found >= 0 ? sm.found : 0;
}

// ------------------------------------------------------------------------ beam top-k
// One CTA per batch row; candidates are beams*V scores. k is small (2 x beam size), so every
// thread keeps its own sorted top-k in registers/local memory and the CTA merges them by k rounds
// of arg-max.
constexpr int TOPK_THREADS = 512;
constexpr int TOPK_MAX = 32;

__global__ void __launch_bounds__(TOPK_THREADS, 1)
beam_topk_kernel(const float* __restrict__ lprobs, const float* __restrict__ beam_scores, float* __restrict__ out_s,
                 long long* __restrict__ out_i, int beams, int V, int k) {
    __shared__ float s_val[TOPK_THREADS / 32];
    __shared__ long long s_idx[TOPK_THREADS / 32];
    __shared__ long long s_win;
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long total = static_cast<long long>(beams) * V;
    const float* base = lprobs + static_cast<size_t>(b) * beams * V;
    float tv[TOPK_MAX];
    long long ti[TOPK_MAX];
#pragma unroll
    for (int j = 0; j < TOPK_MAX; ++j) {
        tv[j] = -FLT_MAX;
        ti[j] = -1;
    }
    float floor_v = -FLT_MAX;   // smallest value in the thread-local top-k once it is full
    int filled = 0;
    for (long long i = tid; i < total; i += TOPK_THREADS) {
        const int beam = static_cast<int>(i / V);
        float v = base[i] + beam_scores[b * beams + beam];
        if (!(v == v)) v = -FLT_MAX;   // NaN never wins
        if (filled < k || v > floor_v) {
            // insertion into the descending list
            int pos = filled < k ? filled : k - 1;
            while (pos > 0 && tv[pos - 1] < v) {
                tv[pos] = tv[pos - 1];
                ti[pos] = ti[pos - 1];
                --pos;
            }
            tv[pos] = v;
            ti[pos] = i;
            if (filled < k) ++filled;
            if (filled == k) floor_v = tv[k - 1];
        }
    }
    int head = 0;   // next unconsumed entry of the local list
    for (int r = 0; r < k; ++r) {
        float v = head < filled ? tv[head] : -FLT_MAX;
        long long idx = head < filled ? ti[head] : -1;
        // arg-max over the CTA, ties broken towards the smaller index for determinism
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const long long oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > v || (ov == v && oi >= 0 && (idx < 0 || oi < idx))) {
                v = ov;
                idx = oi;
            }
        }
        if (lane == 0) {
            s_val[warp] = v;
            s_idx[warp] = idx;
        }
        __syncthreads();
        if (warp == 0) {
            float wv = lane < TOPK_THREADS / 32 ? s_val[lane] : -FLT_MAX;
            long long wi = lane < TOPK_THREADS / 32 ? s_idx[lane] : -1;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, wv, o);
                const long long oi = __shfl_xor_sync(0xffffffffu, wi, o);
                if (ov > wv || (ov == wv && oi >= 0 && (wi < 0 || oi < wi))) {
                    wv = ov;
                    wi = oi;
                }
            }
            if (lane == 0) {
                out_s[b * k + r] = wv;
                out_i[b * k + r] = wi;
                s_win = wi;
            }
        }
        __syncthreads();
        if (head < filled && ti[head] == s_win) ++head;
        __syncthreads();
    }
}

}  // namespace

void ngram_repeat_block(const long long* seqs, float* probs, int batch, int seq_len, int vocab, int n,
                        float ban_value, cudaStream_t st) {
    if (batch == 0 || seq_len < n) return;
    ngram_repeat_block_kernel<<<batch, 256, 0, st>>>(seqs, probs, seq_len, vocab, n, ban_value);
}

void sample_top_p_top_k(const float* probs, const float* uniform, long long* out, int batch, int vocab, float p,
                        int k, cudaStream_t st) {
    if (batch == 0) return;
    static bool configured = false;
    const size_t smem = sizeof(SelSmem);
    if (!configured) {
        cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        configured = true;
    }
    sample_kernel<<<batch, SEL_THREADS, smem, st>>>(probs, uniform, out, vocab, p, k);
}

void beam_topk(const float* lprobs, const float* beam_scores, float* out_scores, long long* out_idx, int batch,
               int beams, int vocab, int k, cudaStream_t st) {
    if (batch == 0) return;
    beam_topk_kernel<<<batch, TOPK_THREADS, 0, st>>>(lprobs, beam_scores, out_scores, out_idx, beams, vocab, k);
}

}  // namespace fs2
