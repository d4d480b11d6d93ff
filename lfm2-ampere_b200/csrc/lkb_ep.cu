// lkb_ep.cu - expert-parallel prefill over NVLink peer memory: the token exchange without a host round trip.
//
// One process per GPU.  Every rank owns four buffers in symmetric memory (same size on every rank, each mapped into
// every peer): the G x G count matrix, three rows of arrival flags, the receive buffer for dispatched rows and the
// buffer its own D rows come back into.  Kernels write straight into a PEER's buffers with ordinary stores over
// NVLink and publish them with a system-scope release store of the layer's epoch into that peer's flag word; the
// consumer polls its OWN flag words (local memory) with acquire loads.  Plain stores only: nothing here goes
// through the switch's reduction or broadcast units, and no bulk-copy engine touches peer memory.  Every wait is bounded: on expiry the kernel records a code in the caller's status word and returns.
//
// Order inside a layer (all on the rank's one stream):
//   route_exchange    ONE CTA: slots grouped by owner rank (stable), advance the epoch (a device int, so the whole step
//                     can be captured in a CUDA graph); my row of the count matrix -> every rank (so every rank knows
//                     who sends how much to whom); wait for all G rows; derive this rank's offsets
//   pack_push         a dispatched slot's 2576-byte row goes straight into its owner's receive buffer at
//                     (rows lower ranks send there) + (its index among my rows for that owner): the owner sees
//                     source-ascending, slot-ascending rows -- the order that makes results bit-identical to 1 GPU
//   route_experts     ONE CTA: wait(rows), then the grouped GEMMs' plan over the received rows (row count read from
//                     device memory), each row's home address and its 1/rms
//   grouped GEMMs     gate|up reads the packed rows; down writes each result row straight to its home rank's return
//                     buffer in that rank's send order
//   publish_wait      phase 2 published, then wait for every source's; then the rank-order combine
// A rank can be at most one phase ahead of its slowest peer, which is what makes buffer reuse across layers safe.
#include "lkb_device.cuh"

#define EP_ROW_BYTES (LKB_HIDDEN + (LKB_HIDDEN / 32) * 8 + 16)        // == LKB_EP_ROW_BYTES
#define EP_MAX_RANKS 8
#define EP_SPIN      (1u << 26)

struct EpPeers {                      // peer views of the four symmetric buffers, indexed by rank
    int *           cmat[EP_MAX_RANKS];
    int *           flags[EP_MAX_RANKS];
    unsigned char * recv[EP_MAX_RANKS];
    float *         dback[EP_MAX_RANKS];
};

__device__ __forceinline__ void ep_st_release(int * p, int v) { asm volatile("st.release.sys.global.s32 [%0], %1;" :: "l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ int ep_ld_acquire(const int * p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ep_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Thread s waits until flags[phase][s] reaches epoch.  The wait ends after limit_ns (and, should the timer stand
// still, after EP_SPIN polls): it then records `code` in *status and returns false; a code already there ends it too.
__device__ __forceinline__ bool ep_wait_flag(const int * flags, int phase, int s, int epoch, int * status, int code,
                                             unsigned long long limit_ns) {
    const int * f = flags + phase * EP_MAX_RANKS + s;
    const unsigned long long t0 = ep_now_ns();
    for (unsigned i = 0; i < EP_SPIN; ++i) {
        if (ep_ld_acquire(f) >= epoch) return true;
        if ((i & 63u) == 63u) {
            if (*(volatile int *) status != 0) return false;
            if (ep_now_ns() - t0 > limit_ns) break;
        }
    }
    atomicCAS(status, 0, code);
    return false;
}

// offs layout (ints): [0, G) send_base[g]: first row of mine inside rank g's receive buffer
//                     [G, 2G) recv_off[s]: first row of source s inside my receive buffer
//                     [2G, 3G) back_base[s]: first row of my block inside source s's return buffer (its send order)
//                     [3G] n_recv
// Row p of my send order (slot send_order[p], destination rank = its expert's owner) -> the owner's receive buffer.
// doff[g] = first position of destination g in my send order.  A warp per row, rows walked with a grid stride by a grid
// of a few CTAs per SM, ONE system-scope fence per CTA at the end (a fence per row made the kernel wait for the NVLink
// round trip 2048 times); the last CTA to finish publishes the rows.
__global__ void __launch_bounds__(256) k_ep_pack_push(const int8_t * __restrict__ aqs, const float2 * __restrict__ asc,
                                                      const float * __restrict__ inv, const int * __restrict__ idx,
                                                      const int * __restrict__ send_order, const int * __restrict__ doff,
                                                      const int * __restrict__ offs, int n, int experts_per_rank, EpPeers P, int me, int G,
                                                      const int * __restrict__ epoch_dev, int * __restrict__ pos,
                                                      unsigned * __restrict__ done) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int p = blockIdx.x * 8 + warp; p < n; p += gridDim.x * 8) {
        const int slot = send_order[p], t = slot >> 2;
        const int e = idx[slot], dest = e / experts_per_rank;
        uint4 * row = reinterpret_cast<uint4 *>(P.recv[dest] + (size_t) (offs[dest] + p - doff[dest]) * EP_ROW_BYTES);
        const uint4 * q = reinterpret_cast<const uint4 *>(aqs + (size_t) t * LKB_HIDDEN);
        const uint4 * sc = reinterpret_cast<const uint4 *>(asc + (size_t) t * (LKB_HIDDEN / 32));
        const uint4 v0 = q[lane], v1 = q[lane + 32], v2 = q[lane + 64], v3 = q[lane + 96], v4 = sc[lane];
        row[lane] = v0; row[lane + 32] = v1; row[lane + 64] = v2; row[lane + 96] = v3; row[lane + 128] = v4;
        if (lane == 0) {
            row[160] = make_uint4(__float_as_uint(inv[t]), (unsigned) (e % experts_per_rank), 0u, 0u);
            pos[slot] = p;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(done, 1u) == gridDim.x - 1) {
        *done = 0u;
        __threadfence_system();
        const int epoch = *epoch_dev;
        for (int g = 0; g < G; ++g) ep_st_release(P.flags[g] + 1 * EP_MAX_RANKS + me, epoch);
    }
}

// Wait until every source has published `phase` for this epoch.
__global__ void __launch_bounds__(32) k_ep_wait(const int * __restrict__ flags, int phase, int G, const int * __restrict__ epoch_dev,
                                                int * __restrict__ status, unsigned long long limit_ns) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    const int epoch = *epoch_dev;
    if ((int) threadIdx.x < G) ep_wait_flag(flags, phase, threadIdx.x, epoch, status, 2 + phase, limit_ns);
}

// ---------------------------------------------------------------------------
// One-CTA routing: histogram of n keys in [0, 64), exclusive offsets, optional 64-row tiles in key order (the
// grouped GEMM's plan), and the stable scatter perm (key-major, index-ascending inside a key) -- the results of the
// count / plan / scatter kernels of the single-GPU path in ONE launch of 1024 threads.  A rank's share of a chunk is a
// few thousand slots, for which four launches cost more than the work; chunks of 1024 keys are ranked with match_any
// and a per-warp count table, with a running offset per key carried from chunk to chunk.
// ---------------------------------------------------------------------------
struct EpRouteSmem { int wc[32][LKB_N_EXPERTS]; int cnt[LKB_N_EXPERTS]; int run[LKB_N_EXPERTS]; int ok; };

template <class KeyFn>
__device__ __forceinline__ void ep_route_cta(EpRouteSmem & R, KeyFn key, int n, int * __restrict__ cnt_out, int * __restrict__ off,
                                             int4 * __restrict__ tiles, int * __restrict__ ntiles, int * __restrict__ perm) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < LKB_N_EXPERTS) R.cnt[tid] = 0;
    __syncthreads();
    for (int s = tid; s < n; s += 1024) atomicAdd(&R.cnt[key(s)], 1);
    __syncthreads();
    if (warp == 0) {
        const int c0 = R.cnt[lane], c1 = R.cnt[lane + 32];
        const int n0 = (c0 + LKB_MOE_BN - 1) / LKB_MOE_BN, n1 = (c1 + LKB_MOE_BN - 1) / LKB_MOE_BN;
        int so = c0, st = n0, so1 = c1, st1 = n1;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int a = __shfl_up_sync(LKB_FULL, so, o), b = __shfl_up_sync(LKB_FULL, st, o);
            const int c = __shfl_up_sync(LKB_FULL, so1, o), d = __shfl_up_sync(LKB_FULL, st1, o);
            if (lane >= o) { so += a; st += b; so1 += c; st1 += d; }
        }
        const int tot_o = __shfl_sync(LKB_FULL, so, 31), tot_t = __shfl_sync(LKB_FULL, st, 31);
        const int off0 = so - c0, off1 = tot_o + so1 - c1;
        R.run[lane] = off0; R.run[lane + 32] = off1;
        off[lane] = off0; off[lane + 32] = off1;
        if (cnt_out) { cnt_out[lane] = c0; cnt_out[lane + 32] = c1; }
        if (tiles) {
            const int tb0 = st - n0, tb1 = tot_t + st1 - n1;
            for (int i = 0; i < n0; ++i) tiles[tb0 + i] = make_int4(lane, off0 + i * LKB_MOE_BN, min(LKB_MOE_BN, c0 - i * LKB_MOE_BN), 0);
            for (int i = 0; i < n1; ++i) tiles[tb1 + i] = make_int4(lane + 32, off1 + i * LKB_MOE_BN, min(LKB_MOE_BN, c1 - i * LKB_MOE_BN), 0);
            if (lane == 31) *ntiles = tot_t + st1;
        }
    }
    for (int c0 = 0; c0 < n; c0 += 1024) {
        for (int i = tid; i < 32 * LKB_N_EXPERTS; i += 1024) (&R.wc[0][0])[i] = 0;
        __syncthreads();
        const int s = c0 + tid;
        const bool live = s < n;
        const int e = live ? key(s) : -1 - lane;               // dead lanes match nobody
        const unsigned same = __match_any_sync(LKB_FULL, e);
        const int rank_w = __popc(same & ((1u << lane) - 1u));
        if (live && rank_w == 0) R.wc[warp][e] = __popc(same);
        __syncthreads();
        if (tid < LKB_N_EXPERTS) {                             // exclusive scan over the 32 warps, per key, from the running offset
            int run = R.run[tid];
            for (int wv = 0; wv < 32; ++wv) { const int c = R.wc[wv][tid]; R.wc[wv][tid] = run; run += c; }
            R.run[tid] = run;
        }
        __syncthreads();
        if (live) perm[R.wc[warp][e] + rank_w] = s;
        __syncthreads();
    }
}

// Home side of a layer's exchange in one launch: slots grouped by the rank that owns their expert (send_order, doff),
// then the count exchange: my row of the G x G count matrix -> every rank, wait for all rows, derive this rank's offsets.
__global__ void __launch_bounds__(1024) k_ep_route_exchange(const int * __restrict__ idx, int ns, int experts_per_rank, EpPeers P, int me, int G,
                                                            int * __restrict__ epoch_dev, int * __restrict__ send_order, int * __restrict__ doff,
                                                            int * __restrict__ offs, int * __restrict__ status, unsigned long long limit_ns) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    __shared__ EpRouteSmem R;
    const int t = threadIdx.x;
    ep_route_cta(R, [&](int s) { return idx[s] / experts_per_rank; }, ns, nullptr, doff, nullptr, nullptr, send_order);
    const int epoch = *epoch_dev + 1;                                    // this layer's epoch; stored back at the end
    if (t < G * G) P.cmat[t / G][me * G + (t % G)] = R.cnt[t % G];      // my row, into every rank's matrix
    __threadfence_system();
    if (t == 0) R.ok = 1;
    __syncthreads();
    if (t < G) ep_st_release(P.flags[t] + 0 * EP_MAX_RANKS + me, epoch);
    if (t < G && !ep_wait_flag(P.flags[me], 0, t, epoch, status, 1, limit_ns)) R.ok = 0;
    __syncthreads();
    if (!R.ok) return;
    const int * C = P.cmat[me];                                          // my copy: C[s*G + g] = rows s sends to g
    if (t < G) {
        int sb = 0, ro = 0, bb = 0;
        for (int s = 0; s < me; ++s) sb += __ldcg(C + s * G + t);
        for (int s = 0; s < t; ++s) ro += __ldcg(C + s * G + me);
        for (int g = 0; g < me; ++g) bb += __ldcg(C + t * G + g);
        offs[t] = sb; offs[G + t] = ro; offs[2 * G + t] = bb;
    }
    if (t == 0) {
        int n = 0;
        for (int s = 0; s < G; ++s) n += __ldcg(C + s * G + me);
        offs[3 * G] = n;
        *epoch_dev = epoch;
    }
}

// Owner side in one launch: wait until every source has published its rows, then the grouped GEMM's plan over the
// received rows (key = the local expert id each row carries).
__global__ void __launch_bounds__(1024) k_ep_route_experts(const unsigned char * __restrict__ recv, int cap, const int * __restrict__ flags, int G,
                                                           const int * __restrict__ epoch_dev, const int * __restrict__ offs,
                                                           int * __restrict__ cnt, int * __restrict__ off, int4 * __restrict__ tiles,
                                                           int * __restrict__ ntiles, int * __restrict__ perm, int * __restrict__ nrecv_out,
                                                           EpPeers P, float ** __restrict__ home_rows, float * __restrict__ inv_out,
                                                           int * __restrict__ status, unsigned long long limit_ns) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    __shared__ EpRouteSmem R;
    const int t = threadIdx.x;
    if (t == 0) R.ok = 1;
    __syncthreads();
    if (t < G && !ep_wait_flag(flags, 1, t, *epoch_dev, status, 3, limit_ns)) R.ok = 0;
    __syncthreads();
    if (!R.ok) { if (t == 0) *ntiles = 0; return; }          // nothing for the GEMMs to do
    int n = offs[3 * G]; if (n > cap) n = cap;
    ep_route_cta(R, [&](int s) { return (int) __ldcg(reinterpret_cast<const unsigned *>(recv + (size_t) s * EP_ROW_BYTES) + 641); },
                 n, cnt, off, tiles, ntiles, perm);
    if (t == 0 && nrecv_out) *nrecv_out = n;
    // the rows' 1/rms as a plane of its own (the grouped GEMM's per-row scale), for callers that feed the GEMM the packed rows
    if (inv_out)
        for (int r = t; r < n; r += 1024) inv_out[r] = __uint_as_float(__ldcg(reinterpret_cast<const unsigned *>(recv + (size_t) r * EP_ROW_BYTES) + 640));
    // where each received row's result goes home to: row (back_base[s] + j) of source s's return buffer (its send order)
    if (home_rows) {
        for (int r = t; r < n; r += 1024) {
            int s = 0;
            while (s + 1 < G && r >= offs[G + s + 1]) ++s;
            home_rows[r] = P.dback[s] + (size_t) (offs[2 * G + s] + (r - offs[G + s])) * LKB_HIDDEN;
        }
    }
}

// Publish `phase` of this epoch to every rank: the stores of the kernels before this one on the stream (the grouped
// GEMM writing result rows straight into their home ranks' buffers) are complete when this kernel starts.
__global__ void __launch_bounds__(32) k_ep_publish(EpPeers P, int me, int G, int phase, const int * __restrict__ epoch_dev,
                                                   const int * __restrict__ wait_flags, int * __restrict__ status, unsigned long long limit_ns) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    __threadfence_system();
    const int epoch = *epoch_dev;
    if ((int) threadIdx.x < G) ep_st_release(P.flags[threadIdx.x] + phase * EP_MAX_RANKS + me, epoch);
    // optionally the wait for the same phase of every source in the same launch (lkb_ep_wait's job)
    if (wait_flags && (int) threadIdx.x < G) ep_wait_flag(wait_flags, phase, threadIdx.x, epoch, status, 2 + phase, limit_ns);
}

static int ep_peers(EpPeers & P, const void * const * cmat, const void * const * flags, const void * const * recv,
                    const void * const * dback, int G) {
    if (!cmat || !flags || !recv || !dback) return LKB_ERR_NULL;
    if (G < 1 || G > EP_MAX_RANKS) return LKB_ERR_SHAPE;
    for (int g = 0; g < G; ++g) {
        if (!cmat[g] || !flags[g] || !recv[g] || !dback[g]) return LKB_ERR_NULL;
        P.cmat[g] = (int *) cmat[g]; P.flags[g] = (int *) flags[g]; P.recv[g] = (unsigned char *) recv[g]; P.dback[g] = (float *) dback[g];
    }
    return LKB_OK;
}

static unsigned long long g_ep_limit_ns = 5000ull * 1000000ull;

extern "C" {

int lkb_ep_set_wait_limit_ms(int ms) {
    if (ms <= 0 || ms > 60000) return LKB_ERR_SHAPE;
    g_ep_limit_ns = (unsigned long long) ms * 1000000ull;
    return LKB_OK;
}

int lkb_ep_route_exchange(const int * idx, int n, int experts_per_rank, const lkb_ep_peers * peers, int me, int G, int * epoch,
                          int * send_order, int * doff, int * offs, int * status, lkb_stream_t st) {
    if (!lkb_context().inited) return LKB_ERR_NOT_INIT;
    if (!idx || !peers || !epoch || !send_order || !doff || !offs || !status) return LKB_ERR_NULL;
    EpPeers P = {};
    const int r = ep_peers(P, peers->cmat, peers->flags, peers->recv, peers->dback, G);
    if (r != LKB_OK) return r;
    if (n <= 0 || experts_per_rank <= 0 || me < 0 || me >= G) return LKB_ERR_SHAPE;
    LKB_PF_LAUNCH(k_ep_route_exchange, dim3(1), dim3(1024), 0, (cudaStream_t) st, idx, n, experts_per_rank, P, me, G, epoch, send_order, doff, offs, status, g_ep_limit_ns);
    return lkb_check_launch();
}

int lkb_ep_route_experts(const void * recv, int cap, const int * flags, int G, const int * epoch, const int * offs, int * cnt, int * off,
                         int * tiles, int * ntiles, int * perm, int * nrecv_out, const lkb_ep_peers * peers, float ** home_rows,
                         float * inv_out, int * status, lkb_stream_t st) {
    if (!lkb_context().inited) return LKB_ERR_NOT_INIT;
    if (!recv || !flags || !epoch || !offs || !cnt || !off || !tiles || !ntiles || !perm || !status) return LKB_ERR_NULL;
    if (cap <= 0 || G < 1 || G > EP_MAX_RANKS) return LKB_ERR_SHAPE;
    EpPeers P = {};
    if (home_rows) {
        if (!peers) return LKB_ERR_NULL;
        const int r = ep_peers(P, peers->cmat, peers->flags, peers->recv, peers->dback, G);
        if (r != LKB_OK) return r;
    }
    LKB_PF_LAUNCH(k_ep_route_experts, dim3(1), dim3(1024), 0, (cudaStream_t) st, reinterpret_cast<const unsigned char *>(recv), cap, flags, G, epoch, offs, cnt, off,
                                                          reinterpret_cast<int4 *>(tiles), ntiles, perm, nrecv_out, P, home_rows, inv_out, status,
                                                          g_ep_limit_ns);
    return lkb_check_launch();
}

int lkb_ep_publish_wait(const lkb_ep_peers * peers, int me, int G, int phase, const int * epoch, const int * flags, int * status,
                        lkb_stream_t st) {
    if (!lkb_context().inited) return LKB_ERR_NOT_INIT;
    if (!peers || !epoch || !flags || !status) return LKB_ERR_NULL;
    EpPeers P = {};
    const int r = ep_peers(P, peers->cmat, peers->flags, peers->recv, peers->dback, G);
    if (r != LKB_OK) return r;
    if (me < 0 || me >= G || phase < 0 || phase > 2) return LKB_ERR_SHAPE;
    LKB_PF_LAUNCH(k_ep_publish, dim3(1), dim3(32), 0, (cudaStream_t) st, P, me, G, phase, epoch, flags, status, g_ep_limit_ns);
    return lkb_check_launch();
}

int lkb_ep_pack_push(lkb_pf_act a, const float * inv, const int * idx, const int * send_order, const int * doff, const int * offs,
                     int n, int experts_per_rank, const lkb_ep_peers * peers, int me, int G, const int * epoch, int * pos, unsigned * done,
                     lkb_stream_t st) {
    if (!lkb_context().inited) return LKB_ERR_NOT_INIT;
    if (!a.qs || !a.sc || !inv || !idx || !send_order || !doff || !offs || !peers || !epoch || !pos || !done) return LKB_ERR_NULL;
    EpPeers P = {};
    const int r = ep_peers(P, peers->cmat, peers->flags, peers->recv, peers->dback, G);
    if (r != LKB_OK) return r;
    if (n <= 0 || experts_per_rank <= 0 || me < 0 || me >= G) return LKB_ERR_SHAPE;
    int grid = lkb_context().sm_count * 4;
    if (grid > (n + 7) / 8) grid = (n + 7) / 8;
    LKB_PF_LAUNCH(k_ep_pack_push, dim3(grid), dim3(256), 0, (cudaStream_t) st, reinterpret_cast<const int8_t *>(a.qs), reinterpret_cast<const float2 *>(a.sc), inv,
                                                        idx, send_order, doff, offs, n, experts_per_rank, P, me, G, epoch, pos, done);
    return lkb_check_launch();
}

int lkb_ep_wait(const int * flags, int phase, int G, const int * epoch, int * status, lkb_stream_t st) {
    if (!lkb_context().inited) return LKB_ERR_NOT_INIT;
    if (!flags || !epoch || !status) return LKB_ERR_NULL;
    if (phase < 0 || phase > 2 || G < 1 || G > EP_MAX_RANKS) return LKB_ERR_SHAPE;
    LKB_PF_LAUNCH(k_ep_wait, dim3(1), dim3(32), 0, (cudaStream_t) st, flags, phase, G, epoch, status, g_ep_limit_ns);
    return lkb_check_launch();
}

}  // extern "C"
