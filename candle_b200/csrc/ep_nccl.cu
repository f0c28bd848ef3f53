// Expert parallelism behind the C ABI: one call runs a whole step of the block with the experts sharded over the
// ranks of an NCCL communicator (one process per GPU).
//
// The reference has no multi-device form of this block; its multi-process example shows the plumbing a candle host
// uses (candle-examples/examples/llama_multiprocess/main.rs:148-173: rank 0 creates the NCCL id, every rank calls
// `Comm::from_rank`; model.rs:30-90: the collective sits behind the op's interface).  The same split is kept here:
// candle_moe_ep_unique_id / candle_moe_ep_comm_init mirror those two steps and candle_moe_ep_forward hides both
// all-to-alls (grouped ncclSend / ncclRecv on the caller's stream) behind the block's forward.
//
// Rank r owns experts [r E/N, (r+1) E/N) and routes its own T rows.  What travels forward is the QUANTIZED row (int8
// values, block sums, block scales: what `VecDotType::from_float`, k_quants.rs:1898-1902, would produce on the
// receiving side anyway), what travels back is the f32 expert output; results equal the single-device block's.
//
// Two forms, chosen from the configuration alone (so every rank picks the same one without talking):
//   slots  (small steps, e.g. decode): every (source, destination) pair owns a slot of fixed capacity
//          C = max_tokens * min(top_k, local experts) rows; the per-expert counts travel in-band in a slot header and
//          are only ever read on the device.  No host synchronisation, no size depends on the data: the step is a
//          fixed sequence of launches and NCCL calls.
//   exact  (large steps): the counts are exchanged first and read by the host (one stream synchronisation), checked
//          on every rank, the verdict is agreed with an all-reduce BEFORE any row moves (a rank that sees an
//          inconsistent table makes every rank return CANDLE_MOE_E_EP_MISMATCH), then the rows travel with their
//          exact sizes.
// NCCL is loaded at run time (libnccl.so.2, the copy already in the process if there is one); a library user who
// never calls these entry points needs no NCCL.
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "api_internal.cuh"

using namespace cmoe;

namespace {

// ---------------------------------------------------------------------------------------------------------
// NCCL through dlopen
// ---------------------------------------------------------------------------------------------------------
struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*CommAbort)(ncclComm_t);
    ncclResult_t (*CommCount)(const ncclComm_t, int*);
    ncclResult_t (*CommUserRank)(const ncclComm_t, int*);
    ncclResult_t (*GroupStart)();
    ncclResult_t (*GroupEnd)();
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
    const char* (*GetErrorString)(ncclResult_t);
};

thread_local std::string g_ep_error;

const NcclApi* nccl_api() {
    static NcclApi api;
    static const bool ok = [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
        if (!h) return false;
        bool all = true;
        const auto sym = [&](const char* name) {
            void* p = dlsym(h, name);
            all = all && p != nullptr;
            return p;
        };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(sym("ncclCommAbort"));
        api.CommCount = reinterpret_cast<decltype(api.CommCount)>(sym("ncclCommCount"));
        api.CommUserRank = reinterpret_cast<decltype(api.CommUserRank)>(sym("ncclCommUserRank"));
        api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
        api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
        api.Send = reinterpret_cast<decltype(api.Send)>(sym("ncclSend"));
        api.Recv = reinterpret_cast<decltype(api.Recv)>(sym("ncclRecv"));
        api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
        return all;
    }();
    return ok ? &api : nullptr;
}

int nccl_fail(const char* what, ncclResult_t r) {
    const NcclApi* a = nccl_api();
    g_ep_error = std::string(what) + ": " + (a ? a->GetErrorString(r) : "NCCL not loaded");
    return CANDLE_MOE_E_NCCL;
}
#define NC_TRY(call)                                              \
    do {                                                          \
        const ncclResult_t _r = (call);                           \
        if (_r != ncclSuccess) return nccl_fail(#call, _r);       \
    } while (0)
#define CU_TRY(call)                                  \
    do {                                              \
        const cudaError_t _e = (call);                \
        if (_e != cudaSuccess) return (int)_e;        \
    } while (0)

}  // namespace

// The communicator handle of the C ABI: an NCCL communicator plus a little pinned host memory for the one
// device-to-host read of the exact form.
struct candle_moe_ep_comm {
    ncclComm_t comm;
    bool owned;
    int rank, world;
    uint32_t* host;  // pinned
    size_t host_words;
};

namespace {

constexpr uint32_t EP_MAGIC = 0x45504d43u;  // "CMPE"
constexpr size_t SLOT_FORM_MAX_BYTES = (size_t)24 << 20;  // per direction and rank; above it the exact form runs
constexpr int EP_PHASES = 5;  // route + pack, exchange of rows, local experts, exchange of results, combine

struct EpProbe {
    cudaEvent_t ev[EP_PHASES + 1];
    int64_t rows_received, rows_busiest_expert;  // exact form only (the host knows them); -1 otherwise
};
thread_local EpProbe* g_ep_probe = nullptr;
inline void ep_mark(cudaStream_t st, int i) {
    if (g_ep_probe) cudaEventRecord(g_ep_probe->ev[i], st);
}

// what every rank must agree on, folded into one word that travels with the counts
uint32_t fingerprint(const candle_moe_ep_config_t* c, const candle_moe_weights_t* w, uint32_t row_bytes) {
    uint32_t h = 2166136261u;
    const uint32_t v[] = {(uint32_t)c->world, (uint32_t)c->n_experts_global, (uint32_t)c->top_k, (uint32_t)c->max_tokens,
                          (uint32_t)w->d_model, (uint32_t)w->n_experts, row_bytes};
    for (uint32_t x : v) h = (h ^ x) * 16777619u;
    return h;
}

struct EpGeometry {
    int N, rank, E, El, k, d, Tm;
    int C;                 // slot capacity in rows (slot form)
    bool slots;
    uint32_t row_bytes;    // packed quantized row
    uint32_t hdr_bytes;    // slot header: 4 words + El counts, padded to 16 bytes
    size_t slot_bytes;     // header + C rows
    int64_t P_cap;         // bound on the rows a rank may receive in one step
    int msg_words;         // exact form: El counts + 2 words per (source, destination) message
    uint32_t fp;
};

int geometry(const candle_moe_ep_config_t* c, const candle_moe_weights_t* w, EpGeometry& g) {
    if (!c || !w) return CANDLE_MOE_E_NULL;
    CM_TRY(check_weights(w));
    if (w->dtype_w13 == CANDLE_GGML_Q8_0 || w->dtype_w2 == CANDLE_GGML_Q8_0 || w->d_ff_shared > 0) return CANDLE_MOE_E_DTYPE;
    if (c->world <= 0 || c->rank < 0 || c->rank >= c->world || c->max_tokens <= 0 || c->max_tokens > (1 << 22)) return CANDLE_MOE_E_SHAPE;
    if (c->n_experts_global <= 0 || c->n_experts_global > CANDLE_MOE_MAX_EXPERTS || c->n_experts_global % c->world) return CANDLE_MOE_E_SHAPE;
    if (w->n_experts != c->n_experts_global / c->world) return CANDLE_MOE_E_SHAPE;
    if (c->top_k <= 0 || c->top_k > CANDLE_MOE_MAX_TOPK || c->top_k > c->n_experts_global) return CANDLE_MOE_E_SHAPE;
    if (w->d_model % 256 || (int64_t)c->world * w->n_experts > 1024) return CANDLE_MOE_E_SHAPE;
    if (!c->router) return CANDLE_MOE_E_NULL;
    g.N = c->world;
    g.rank = c->rank;
    g.E = c->n_experts_global;
    g.El = w->n_experts;
    g.k = c->top_k;
    g.d = w->d_model;
    g.Tm = c->max_tokens;
    g.row_bytes = (uint32_t)ep_row_bytes(g.d);
    g.hdr_bytes = (uint32_t)align_up(16 + 4 * (size_t)g.El, 16);
    g.C = g.Tm * std::min(g.k, g.El);  // a token selects an expert at most once
    g.slot_bytes = g.hdr_bytes + (size_t)g.C * g.row_bytes;
    const size_t back_bytes = (size_t)g.N * g.C * g.d * 4;
    g.slots = std::max((size_t)g.N * g.slot_bytes, back_bytes) <= SLOT_FORM_MAX_BYTES;
    if (c->force_form == 1) g.slots = true;
    if (c->force_form == 2) g.slots = false;
    g.P_cap = (int64_t)g.N * g.C;
    if (!g.slots && c->max_recv_rows > 0) g.P_cap = std::min<int64_t>(g.P_cap, c->max_recv_rows);
    g.msg_words = g.El + 2;
    g.fp = fingerprint(c, w, g.row_bytes);
    return CANDLE_MOE_OK;
}

struct EpFwdWorkspace {
    uint32_t *ids, *counts, *offsets, *perm, *pair_pos, *slot_pos, *perm_scratch;
    float* tw;
    int8_t* xq;
    float* xs;
    int16_t* xb;
    uint32_t *msg_send, *msg_recv, *recv_counts, *plan;  // plan: [3][1024] in_base, out_base, rows per source
    int32_t* flag;
    uint8_t *send, *recv;
    float *ret_send, *ret_recv;
    void* local;
    size_t local_bytes, total;
};

EpFwdWorkspace fwd_layout(const EpGeometry& g, const candle_moe_weights_t* w, void* base_) {
    uint8_t* base = static_cast<uint8_t*>(base_);
    EpFwdWorkspace ws{};
    size_t off = 0;
    const size_t Tk = (size_t)g.Tm * g.k, d = g.d;
    ws.ids = carve<uint32_t>(base, off, Tk);
    ws.tw = carve<float>(base, off, Tk);
    ws.counts = carve<uint32_t>(base, off, g.E);
    ws.offsets = carve<uint32_t>(base, off, g.E + 1);
    ws.perm = carve<uint32_t>(base, off, Tk);
    ws.pair_pos = carve<uint32_t>(base, off, Tk);
    ws.slot_pos = carve<uint32_t>(base, off, Tk);
    ws.perm_scratch = carve<uint32_t>(base, off, permute_scratch_words((int64_t)Tk, g.E));
    ws.xq = carve<int8_t>(base, off, (size_t)g.Tm * d);
    ws.xs = carve<float>(base, off, (size_t)g.Tm * d / 256);
    ws.xb = carve<int16_t>(base, off, (size_t)g.Tm * d / 16);
    ws.msg_send = carve<uint32_t>(base, off, (size_t)g.N * g.msg_words);
    ws.msg_recv = carve<uint32_t>(base, off, (size_t)g.N * g.msg_words);
    ws.recv_counts = carve<uint32_t>(base, off, (size_t)g.N * g.El);
    ws.plan = carve<uint32_t>(base, off, 3 * 1024);
    ws.flag = carve<int32_t>(base, off, 4);
    if (g.slots) {
        ws.send = carve<uint8_t>(base, off, (size_t)g.N * g.slot_bytes);
        ws.recv = carve<uint8_t>(base, off, (size_t)g.N * g.slot_bytes);
        ws.ret_send = carve<float>(base, off, (size_t)g.N * g.C * d);
        ws.ret_recv = carve<float>(base, off, (size_t)g.N * g.C * d);
    } else {
        ws.send = carve<uint8_t>(base, off, Tk * g.row_bytes);
        ws.recv = carve<uint8_t>(base, off, (size_t)g.P_cap * g.row_bytes);
        ws.ret_send = carve<float>(base, off, (size_t)g.P_cap * d);
        ws.ret_recv = carve<float>(base, off, Tk * d);
    }
    off = align_up(off, 256);
    ws.local_bytes = ep_layout(w, g.P_cap, nullptr).total;
    ws.local = base ? base + off : nullptr;
    off += ws.local_bytes;
    ws.total = align_up(off, 256);
    return ws;
}

// ---------------------------------------------------------------------------------------------------------
// device side of the slot form
// ---------------------------------------------------------------------------------------------------------
// expert that owns grouped position p: the last e with offs[e] <= p (empty experts share their successor's offset,
// and the last of them is the one with rows)
__device__ __forceinline__ int expert_of(const uint32_t* offs, int E, uint32_t p) {
    int lo = 0, hi = E - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (offs[mid] <= p) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// One warp per grouped position: its packed row goes to the slot of the rank that owns its expert.  The last CTA
// writes the slot headers and, for the combine step, where each (token, rank) pair's result will come back.
__global__ void __launch_bounds__(256)
ep_pack_slots_kernel(const uint32_t* __restrict__ offsets, const uint32_t* __restrict__ perm_token,
                     const uint32_t* __restrict__ pair_pos, int Tk, int T, int d, int E, int El, int N, int C,
                     const int8_t* __restrict__ xq, const float* __restrict__ xs, const int16_t* __restrict__ xb,
                     uint8_t* __restrict__ send, size_t slot_bytes, int hdr_bytes, int row_bytes, uint32_t fp,
                     uint32_t* __restrict__ slot_pos) {
    pdl_trigger();
    pdl_wait();
    __shared__ uint32_t s_offs[CANDLE_MOE_MAX_EXPERTS + 1];
    for (int i = threadIdx.x; i <= E; i += blockDim.x) s_offs[i] = offsets[i];
    __syncthreads();
    if (blockIdx.x == gridDim.x - 1) {
        for (int i = threadIdx.x; i < N * (4 + El); i += blockDim.x) {
            const int dst = i / (4 + El), j = i - dst * (4 + El);
            uint32_t v;
            if (j == 0) v = EP_MAGIC ^ fp;
            else if (j == 1) v = (uint32_t)T;
            else if (j == 2) v = s_offs[(dst + 1) * El] - s_offs[dst * El];
            else if (j == 3) v = 0u;
            else v = s_offs[dst * El + (j - 4) + 1] - s_offs[dst * El + (j - 4)];
            reinterpret_cast<uint32_t*>(send + (size_t)dst * slot_bytes)[j] = v;
        }
        for (int i = threadIdx.x; i < Tk; i += blockDim.x) {
            const uint32_t p = pair_pos[i];
            const int dst = expert_of(s_offs, E, p) / El;
            slot_pos[i] = (uint32_t)dst * (uint32_t)C + (p - s_offs[dst * El]);
        }
        return;
    }
    const int lane = threadIdx.x & 31;
    const int64_t p = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (p >= Tk) return;
    const int dst = expert_of(s_offs, E, (uint32_t)p) / El;
    const int64_t row = perm_token[p];
    uint8_t* out = send + (size_t)dst * slot_bytes + hdr_bytes + (size_t)((uint32_t)p - s_offs[dst * El]) * row_bytes;
    const uint4* q = reinterpret_cast<const uint4*>(xq + row * d);
    for (int i = lane; i < d / 16; i += 32) reinterpret_cast<uint4*>(out)[i] = q[i];
    const uint32_t* b = reinterpret_cast<const uint32_t*>(xb + row * (d / 16));
    for (int i = lane; i < d / 32; i += 32) reinterpret_cast<uint32_t*>(out + d)[i] = b[i];
    const float* s = xs + row * (d / 256);
    for (int i = lane; i < d / 256; i += 32) reinterpret_cast<float*>(out + d + d / 8)[i] = s[i];
}

// Reads the N slot headers, checks them, and lays the received rows out by local expert.  A header that fails a
// check counts as an empty slot and raises bit 2 of the library's health word (candle_moe_device_status): the step
// finishes with that source's rows missing instead of indexing with numbers it cannot trust.
//   plan[0][src * El + e]  first row of group (src, e) inside its slot
//   plan[1][src * El + e]  its first position in expert-major order
//   plan[2][src]           rows in the slot
__global__ void __launch_bounds__(1024)
ep_plan_slots_kernel(const uint8_t* __restrict__ recv, size_t slot_bytes, int N, int El, int C, int Tm, uint32_t fp,
                     uint32_t* __restrict__ plan, uint32_t* __restrict__ offsets, uint32_t* __restrict__ counts_out,
                     int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    __shared__ uint32_t s_cnt[1024], s_eoff[CANDLE_MOE_MAX_EXPERTS + 1], s_rows[1024];
    __shared__ int s_ok[1024];
    const int n = N * El;
    for (int src = threadIdx.x; src < N; src += blockDim.x) {
        const uint32_t* h = reinterpret_cast<const uint32_t*>(recv + (size_t)src * slot_bytes);
        bool ok = h[0] == (EP_MAGIC ^ fp) && h[1] <= (uint32_t)Tm && h[2] <= (uint32_t)C;
        if (ok) {
            uint32_t sum = 0;
            for (int e = 0; e < El; ++e) {
                ok = ok && h[4 + e] <= h[1];
                sum += h[4 + e];
            }
            ok = ok && sum == h[2];
        }
        s_ok[src] = ok;
        s_rows[src] = ok ? h[2] : 0u;
        if (!ok) atomicOr(status, 4);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int src = i / El, e = i - src * El;
        s_cnt[i] = s_ok[src] ? reinterpret_cast<const uint32_t*>(recv + (size_t)src * slot_bytes)[4 + e] : 0u;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t run = 0;
        for (int e = 0; e < El; ++e) {
            s_eoff[e] = run;
            for (int s = 0; s < N; ++s) run += s_cnt[s * El + e];
        }
        s_eoff[El] = run;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= El; e += blockDim.x) offsets[e] = s_eoff[e];
    for (int src = threadIdx.x; src < N; src += blockDim.x) plan[2048 + src] = s_rows[src];
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int src = i / El, e = i - src * El;
        uint32_t ib = 0, ob = s_eoff[e];
        for (int e2 = 0; e2 < e; ++e2) ib += s_cnt[src * El + e2];
        for (int s2 = 0; s2 < src; ++s2) ob += s_cnt[s2 * El + e];
        plan[i] = ib;
        plan[1024 + i] = ob;
        counts_out[i] = s_cnt[i];
    }
}

// one warp per slot row (src, i): unpack into the planar arrays at its expert-major position
__global__ void __launch_bounds__(256)
ep_regroup_slots_kernel(const uint8_t* __restrict__ recv, size_t slot_bytes, int hdr_bytes, int row_bytes, int N, int El, int C,
                        int d, const uint32_t* __restrict__ plan, const uint32_t* __restrict__ counts,
                        int8_t* __restrict__ xq, float* __restrict__ xs, int16_t* __restrict__ xb,
                        uint32_t* __restrict__ back_index) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= (int64_t)N * C) return;
    const int src = (int)(r / C);
    const uint32_t i = (uint32_t)(r - (int64_t)src * C);
    if (i >= plan[2048 + src]) return;
    int e = -1;
    for (int e0 = 0; e0 < El && e < 0; e0 += 32) {
        const int ee = e0 + lane;
        bool hit = false;
        if (ee < El) {
            const uint32_t ib = plan[src * El + ee];
            hit = i >= ib && i < ib + counts[src * El + ee];
        }
        const uint32_t m = __ballot_sync(0xffffffffu, hit);
        if (m) e = e0 + __ffs(m) - 1;
    }
    if (e < 0) return;
    const int64_t p = (int64_t)plan[1024 + src * El + e] + (i - plan[src * El + e]);
    const uint8_t* in = recv + (size_t)src * slot_bytes + hdr_bytes + (size_t)i * row_bytes;
    uint4* q = reinterpret_cast<uint4*>(xq + p * d);
    for (int j = lane; j < d / 16; j += 32) q[j] = reinterpret_cast<const uint4*>(in)[j];
    uint32_t* b = reinterpret_cast<uint32_t*>(xb + p * (d / 16));
    for (int j = lane; j < d / 32; j += 32) b[j] = reinterpret_cast<const uint32_t*>(in + d)[j];
    float* s = xs + p * (d / 256);
    for (int j = lane; j < d / 256; j += 32) s[j] = reinterpret_cast<const float*>(in + d + d / 8)[j];
    if (lane == 0) back_index[p] = (uint32_t)r;
}

// exact form: the (source, destination) messages that carry the counts: [El counts | magic ^ fingerprint | T]
__global__ void __launch_bounds__(256)
ep_count_msgs_kernel(const uint32_t* __restrict__ counts, int N, int El, int T, uint32_t fp, uint32_t* __restrict__ msgs) {
    pdl_trigger();
    pdl_wait();
    const int mw = El + 2;
    for (int i = threadIdx.x; i < N * mw; i += blockDim.x) {
        const int dst = i / mw, j = i - dst * mw;
        msgs[i] = j < El ? counts[dst * El + j] : (j == El ? (EP_MAGIC ^ fp) : (uint32_t)T);
    }
}

// grouped send / receive of equally sized pieces between all ranks; the piece for this rank is a device copy
int exchange_fixed(const NcclApi* a, candle_moe_ep_comm* cm, cudaStream_t st, const uint8_t* send, uint8_t* recv, size_t piece) {
    const int N = cm->world, me = cm->rank;
    CU_TRY(cudaMemcpyAsync(recv + (size_t)me * piece, send + (size_t)me * piece, piece, cudaMemcpyDeviceToDevice, st));
    if (N == 1) return CANDLE_MOE_OK;
    NC_TRY(a->GroupStart());
    for (int i = 1; i < N; ++i) {
        const int to = (me + i) % N, from = (me - i + N) % N;
        NC_TRY(a->Send(send + (size_t)to * piece, piece, ncclUint8, to, cm->comm, st));
        NC_TRY(a->Recv(recv + (size_t)from * piece, piece, ncclUint8, from, cm->comm, st));
    }
    NC_TRY(a->GroupEnd());
    return CANDLE_MOE_OK;
}

// the same with per-peer sizes; pieces are contiguous in rank order on both sides
int exchange_var(const NcclApi* a, candle_moe_ep_comm* cm, cudaStream_t st, const uint8_t* send, const std::vector<size_t>& send_bytes,
                 uint8_t* recv, const std::vector<size_t>& recv_bytes) {
    const int N = cm->world, me = cm->rank;
    std::vector<size_t> so(N + 1, 0), ro(N + 1, 0);
    for (int i = 0; i < N; ++i) {
        so[i + 1] = so[i] + send_bytes[i];
        ro[i + 1] = ro[i] + recv_bytes[i];
    }
    if (send_bytes[me] != recv_bytes[me]) return CANDLE_MOE_E_EP_MISMATCH;
    if (send_bytes[me]) CU_TRY(cudaMemcpyAsync(recv + ro[me], send + so[me], send_bytes[me], cudaMemcpyDeviceToDevice, st));
    if (N == 1) return CANDLE_MOE_OK;
    NC_TRY(a->GroupStart());
    for (int i = 1; i < N; ++i) {
        const int to = (me + i) % N, from = (me - i + N) % N;
        if (send_bytes[to]) NC_TRY(a->Send(send + so[to], send_bytes[to], ncclUint8, to, cm->comm, st));
        if (recv_bytes[from]) NC_TRY(a->Recv(recv + ro[from], recv_bytes[from], ncclUint8, from, cm->comm, st));
    }
    NC_TRY(a->GroupEnd());
    return CANDLE_MOE_OK;
}

int ep_forward_impl(cudaStream_t st, candle_moe_ep_comm* cm, const candle_moe_ep_config_t* cfg, const candle_moe_weights_t* w,
                    const float* x, int64_t T, float* y, void* workspace, size_t workspace_bytes) {
    EpGeometry g;
    CM_TRY(geometry(cfg, w, g));
    if (T < 0 || T > g.Tm) return CANDLE_MOE_E_SHAPE;
    if (!workspace || (T > 0 && (!x || !y))) return CANDLE_MOE_E_NULL;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(y) & 15) ||
        (reinterpret_cast<uintptr_t>(cfg->router) & 15))
        return CANDLE_MOE_E_ALIGN;
    const NcclApi* a = nullptr;
    if (g.N > 1) {
        if (!cm || !cm->comm) return CANDLE_MOE_E_NULL;
        if (cm->world != g.N || cm->rank != g.rank) return CANDLE_MOE_E_SHAPE;
        a = nccl_api();
        if (!a) {
            g_ep_error = "libnccl.so.2 could not be loaded";
            return CANDLE_MOE_E_NCCL;
        }
    }
    candle_moe_ep_comm self{nullptr, false, 0, 1, nullptr, 0};
    if (g.N == 1 && !cm) cm = &self;
    const EpFwdWorkspace ws = fwd_layout(g, w, workspace);
    if (workspace_bytes < ws.total) return CANDLE_MOE_E_WORKSPACE;
    const EpWorkspace lw = ep_layout(w, g.P_cap, ws.local);
    ExpertPtrs p1, p3, p2;
    CM_TRY(fill_ptrs(w->w1, g.El, p1));
    CM_TRY(fill_ptrs(w->w3, g.El, p3));
    CM_TRY(fill_ptrs(w->w2, g.El, p2));
    const int d = g.d, k = g.k, E = g.E, El = g.El, N = g.N;
    const int64_t Tk = T * k;
    int* status = nullptr;
    CU_TRY(stream_status_ptr(&status));

    // ---- route, quantize, group (as on one device; the dispatch order is also destination order) ----
    ep_mark(st, 0);
    if (T > 0) {
        CU_TRY(launch_router_topk(st, x, cfg->router, cfg->router_bias, T, d, E, k, cfg->renorm, ws.ids, ws.tw, ws.xq, ws.xs, ws.xb));
    }
    // with no rows the dispatch still has to say so: counts and offsets of zero
    CU_TRY(launch_permute(st, ws.ids, T, k, E, ws.counts, ws.offsets, ws.perm, ws.pair_pos, ws.perm_scratch));

    int eo_splits = 1;
    if (g.slots) {
        const unsigned grid = (unsigned)((Tk + 7) / 8) + 1;
        // tests: this rank's slot headers carry a wrong check word, so every receiver drops its rows and says so
        const uint32_t fp_send = cfg->inject_count_mismatch == 1 ? g.fp ^ 0x5a5a5a5au : g.fp;
        CU_TRY(launch_k(ep_pack_slots_kernel, dim3(grid), dim3(256), 0, st, (const uint32_t*)ws.offsets, (const uint32_t*)ws.perm,
                        (const uint32_t*)ws.pair_pos, (int)Tk, (int)T, d, E, El, N, g.C, (const int8_t*)ws.xq, (const float*)ws.xs,
                        (const int16_t*)ws.xb, ws.send, g.slot_bytes, (int)g.hdr_bytes, (int)g.row_bytes, fp_send, ws.slot_pos));
        ep_mark(st, 1);
        CM_TRY(exchange_fixed(a, cm, st, ws.send, ws.recv, g.slot_bytes));
        ep_mark(st, 2);
        CU_TRY(launch_k(ep_plan_slots_kernel, dim3(1), dim3(1024), 0, st, (const uint8_t*)ws.recv, g.slot_bytes, N, El, g.C, g.Tm, g.fp,
                        ws.plan, lw.offsets, ws.recv_counts, status));
        CU_TRY(launch_k(ep_regroup_slots_kernel, dim3((unsigned)((g.P_cap + 7) / 8)), dim3(256), 0, st, (const uint8_t*)ws.recv,
                        g.slot_bytes, (int)g.hdr_bytes, (int)g.row_bytes, N, El, g.C, d, (const uint32_t*)ws.plan,
                        (const uint32_t*)ws.recv_counts, lw.xq, lw.xs, lw.xb, lw.back));
        // kernels and tile widths are chosen for five quarters of the EXPECTED rows of an expert under even routing
        // (an expert with a few rows more than the average must not spill into a second, almost empty tile); any
        // count is handled
        const int64_t expect = std::max<int64_t>(1, ((int64_t)N * g.Tm * k + E - 1) / E);
        const int64_t bound = (5 * expect + 3) / 4;
        const int slots_k = ep_eo_slots(g.P_cap, El);
        CM_TRY(run_experts(st, w, p1, p3, p2, bound, g.P_cap, lw.offsets, nullptr, lw.xq, lw.xs, lw.xb, lw.eb, slots_k, &eo_splits,
                           false, true, lw.offsets + El, expect * El));
        CU_TRY(launch_ep_scatter(st, lw.eb.eo, eo_splits, g.P_cap * d, lw.back, g.P_cap, d, ws.ret_send, lw.offsets + El));
        ep_mark(st, 3);
        CM_TRY(exchange_fixed(a, cm, st, reinterpret_cast<const uint8_t*>(ws.ret_send), reinterpret_cast<uint8_t*>(ws.ret_recv),
                              (size_t)g.C * d * 4));
        ep_mark(st, 4);
        if (T > 0)
            CU_TRY(launch_combine(st, ws.ret_recv, 1, 0, ws.ids, ws.tw, ws.slot_pos, T, k, d, nullptr, 1, 0, x, nullptr, y));
        ep_mark(st, 5);
        return CANDLE_MOE_OK;
    }

    // ---------------- exact form ----------------
    if (!cm->host && N > 1) return CANDLE_MOE_E_NULL;
    std::vector<uint32_t> stage_local;
    uint32_t* host = cm->host;
    const size_t need_words = 2 * (size_t)N * g.msg_words + 8;
    if (!host) {  // single rank without a communicator: plain host memory will do (the copies below are synchronous then)
        stage_local.resize(need_words);
        host = stage_local.data();
    } else if (cm->host_words < need_words) {
        return CANDLE_MOE_E_WORKSPACE;
    }
    if (Tk > 0) CU_TRY(launch_ep_pack(st, ws.perm, Tk, d, ws.xq, ws.xs, ws.xb, ws.send));
    CU_TRY(launch_k(ep_count_msgs_kernel, dim3(1), dim3(256), 0, st, (const uint32_t*)ws.counts, N, El, (int)T, g.fp, ws.msg_send));
    ep_mark(st, 1);
    CM_TRY(exchange_fixed(a, cm, st, reinterpret_cast<const uint8_t*>(ws.msg_send), reinterpret_cast<uint8_t*>(ws.msg_recv),
                          (size_t)g.msg_words * 4));
    uint32_t* h_send = host;
    uint32_t* h_recv = host + (size_t)N * g.msg_words;
    int32_t* h_flag = reinterpret_cast<int32_t*>(host + 2 * (size_t)N * g.msg_words);
    CU_TRY(cudaMemcpyAsync(h_send, ws.msg_send, (size_t)N * g.msg_words * 4, cudaMemcpyDeviceToHost, st));
    CU_TRY(cudaMemcpyAsync(h_recv, ws.msg_recv, (size_t)N * g.msg_words * 4, cudaMemcpyDeviceToHost, st));
    CU_TRY(cudaStreamSynchronize(st));  // the one host read of the step

    // ---- every rank checks what it holds; the verdict is agreed before any row moves ----
    std::vector<size_t> send_rows(N), recv_rows(N);
    std::vector<uint32_t> dense((size_t)N * El);
    int64_t n_recv = 0, sent = 0;
    bool ok = true;
    for (int r = 0; r < N; ++r) {
        const uint32_t* ms = h_send + (size_t)r * g.msg_words;
        const uint32_t* mr = h_recv + (size_t)r * g.msg_words;
        size_t s = 0, q = 0;
        for (int e = 0; e < El; ++e) {
            s += ms[e];
            q += mr[e];
            dense[(size_t)r * El + e] = mr[e];
            ok = ok && mr[e] <= mr[El + 1];  // a token selects an expert at most once
        }
        ok = ok && mr[El] == (EP_MAGIC ^ g.fp) && mr[El + 1] <= (uint32_t)g.Tm;
        send_rows[r] = s;
        recv_rows[r] = q;
        sent += (int64_t)s;
        n_recv += (int64_t)q;
    }
    ok = ok && sent == Tk && n_recv <= g.P_cap;
    if (cfg->inject_count_mismatch == 1) ok = false;  // tests: this rank reports a bad table
    if (N > 1) {
        h_flag[0] = ok ? 1 : 0;
        CU_TRY(cudaMemcpyAsync(ws.flag, h_flag, 4, cudaMemcpyHostToDevice, st));
        NC_TRY(a->AllReduce(ws.flag, ws.flag + 1, 1, ncclInt32, ncclMin, cm->comm, st));
        CU_TRY(cudaMemcpyAsync(h_flag + 1, ws.flag + 1, 4, cudaMemcpyDeviceToHost, st));
        CU_TRY(cudaStreamSynchronize(st));
        ok = h_flag[1] != 0;
    }
    if (!ok) {
        g_ep_error = "expert-parallel count tables disagree between ranks (or exceed the configured capacity)";
        return CANDLE_MOE_E_EP_MISMATCH;
    }
    int64_t max_rows = 0;
    for (int e = 0; e < El; ++e) {
        int64_t c = 0;
        for (int r = 0; r < N; ++r) c += dense[(size_t)r * El + e];
        max_rows = std::max(max_rows, c);
    }
    if (g_ep_probe) {
        g_ep_probe->rows_received = n_recv;
        g_ep_probe->rows_busiest_expert = max_rows;
    }
    std::vector<size_t> sb(N), rb(N);
    for (int r = 0; r < N; ++r) {
        sb[r] = send_rows[r] * g.row_bytes;
        rb[r] = recv_rows[r] * g.row_bytes;
    }
    CM_TRY(exchange_var(a, cm, st, ws.send, sb, ws.recv, rb));
    // the dense count table goes back to the device as a kernel-visible array (from the pinned staging area)
    std::memcpy(h_send, dense.data(), dense.size() * 4);
    CU_TRY(cudaMemcpyAsync(ws.recv_counts, h_send, dense.size() * 4, cudaMemcpyHostToDevice, st));
    ep_mark(st, 2);
    if (n_recv > 0) {
        CU_TRY(launch_ep_regroup(st, ws.recv, ws.recv_counts, N, El, n_recv, d, lw.plan, lw.xq, lw.xs, lw.xb, lw.offsets, lw.back));
        const int slots_k = ep_eo_slots(n_recv, El);
        CM_TRY(run_experts(st, w, p1, p3, p2, max_rows, n_recv, lw.offsets, nullptr, lw.xq, lw.xs, lw.xb, lw.eb, slots_k, &eo_splits,
                           false, true, nullptr, 0));
        CU_TRY(launch_ep_scatter(st, lw.eb.eo, eo_splits, n_recv * d, lw.back, n_recv, d, ws.ret_send, nullptr));
    }
    ep_mark(st, 3);
    for (int r = 0; r < N; ++r) {
        sb[r] = recv_rows[r] * (size_t)d * 4;  // what came from r goes back to r
        rb[r] = send_rows[r] * (size_t)d * 4;
    }
    CM_TRY(exchange_var(a, cm, st, reinterpret_cast<const uint8_t*>(ws.ret_send), sb, reinterpret_cast<uint8_t*>(ws.ret_recv), rb));
    ep_mark(st, 4);
    if (T > 0) CU_TRY(launch_combine(st, ws.ret_recv, 1, 0, ws.ids, ws.tw, ws.pair_pos, T, k, d, nullptr, 1, 0, x, nullptr, y));
    ep_mark(st, 5);
    if (!cm->host) CU_TRY(cudaStreamSynchronize(st));  // the pageable staging vector dies with this call
    return CANDLE_MOE_OK;
}

}  // namespace

extern "C" {

const char* candle_moe_ep_last_error(void) { return g_ep_error.c_str(); }

int candle_moe_ep_unique_id(void* id_out) {
    if (!id_out) return CANDLE_MOE_E_NULL;
    const NcclApi* a = nccl_api();
    if (!a) {
        g_ep_error = "libnccl.so.2 could not be loaded";
        return CANDLE_MOE_E_NCCL;
    }
    static_assert(sizeof(ncclUniqueId) == CANDLE_MOE_EP_UNIQUE_ID_BYTES, "id size");
    ncclUniqueId id;
    NC_TRY(a->GetUniqueId(&id));
    std::memcpy(id_out, &id, sizeof(id));
    return CANDLE_MOE_OK;
}

static int make_comm(ncclComm_t c, bool owned, int rank, int world, candle_moe_ep_comm_t** out) {
    auto* cm = new candle_moe_ep_comm{c, owned, rank, world, nullptr, 0};
    cm->host_words = 2 * (size_t)world * (CANDLE_MOE_MAX_EXPERTS + 2) + 64;
    const cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(&cm->host), cm->host_words * 4, cudaHostAllocDefault);
    if (e != cudaSuccess) {
        delete cm;
        return (int)e;
    }
    *out = cm;
    return CANDLE_MOE_OK;
}

int candle_moe_ep_comm_init(const void* unique_id, int32_t rank, int32_t world, candle_moe_ep_comm_t** comm_out) {
    if (!unique_id || !comm_out) return CANDLE_MOE_E_NULL;
    if (world <= 0 || rank < 0 || rank >= world) return CANDLE_MOE_E_SHAPE;
    const NcclApi* a = nccl_api();
    if (!a) {
        g_ep_error = "libnccl.so.2 could not be loaded";
        return CANDLE_MOE_E_NCCL;
    }
    ncclUniqueId id;
    std::memcpy(&id, unique_id, sizeof(id));
    ncclComm_t c = nullptr;
    NC_TRY(a->CommInitRank(&c, world, id, rank));
    const int r = make_comm(c, true, rank, world, comm_out);
    if (r != CANDLE_MOE_OK) a->CommDestroy(c);
    return r;
}

int candle_moe_ep_comm_from_nccl(void* nccl_comm, candle_moe_ep_comm_t** comm_out) {
    if (!nccl_comm || !comm_out) return CANDLE_MOE_E_NULL;
    const NcclApi* a = nccl_api();
    if (!a) {
        g_ep_error = "libnccl.so.2 could not be loaded";
        return CANDLE_MOE_E_NCCL;
    }
    int rank = 0, world = 0;
    NC_TRY(a->CommUserRank(static_cast<ncclComm_t>(nccl_comm), &rank));
    NC_TRY(a->CommCount(static_cast<ncclComm_t>(nccl_comm), &world));
    return make_comm(static_cast<ncclComm_t>(nccl_comm), false, rank, world, comm_out);
}

int candle_moe_ep_comm_destroy(candle_moe_ep_comm_t* cm) {
    if (!cm) return CANDLE_MOE_OK;
    if (cm->host) cudaFreeHost(cm->host);
    int r = CANDLE_MOE_OK;
    if (cm->owned && cm->comm) {
        const NcclApi* a = nccl_api();
        if (a && a->CommDestroy(cm->comm) != ncclSuccess) r = CANDLE_MOE_E_NCCL;
    }
    delete cm;
    return r;
}

int candle_moe_ep_forward_workspace_bytes(const candle_moe_ep_config_t* cfg, const candle_moe_weights_t* local, size_t* out_bytes) {
    if (!out_bytes) return CANDLE_MOE_E_NULL;
    EpGeometry g;
    CM_TRY(geometry(cfg, local, g));
    *out_bytes = fwd_layout(g, local, nullptr).total;
    return CANDLE_MOE_OK;
}

int candle_moe_ep_forward_form(const candle_moe_ep_config_t* cfg, const candle_moe_weights_t* local, int32_t* form, int64_t* capacity_rows) {
    EpGeometry g;
    CM_TRY(geometry(cfg, local, g));
    if (form) *form = g.slots ? 1 : 2;
    if (capacity_rows) *capacity_rows = g.slots ? g.C : g.P_cap;
    return CANDLE_MOE_OK;
}

int candle_moe_ep_forward(void* stream, candle_moe_ep_comm_t* comm, const candle_moe_ep_config_t* cfg,
                          const candle_moe_weights_t* local, const float* x, int64_t T, float* y, void* workspace,
                          size_t workspace_bytes) {
    return ep_forward_impl((cudaStream_t)stream, comm, cfg, local, x, T, y, workspace, workspace_bytes);
}

int candle_moe_ep_forward_timed(void* stream, candle_moe_ep_comm_t* comm, const candle_moe_ep_config_t* cfg,
                                const candle_moe_weights_t* local, const float* x, int64_t T, float* y, void* workspace,
                                size_t workspace_bytes, float* phase_ms, int64_t* rows_info) {
    if (!phase_ms) return CANDLE_MOE_E_NULL;
    EpProbe probe{};
    probe.rows_received = probe.rows_busiest_expert = -1;
    for (int i = 0; i <= EP_PHASES; ++i) {
        const cudaError_t e = cudaEventCreate(&probe.ev[i]);
        if (e != cudaSuccess) {
            for (int j = 0; j < i; ++j) cudaEventDestroy(probe.ev[j]);
            return (int)e;
        }
    }
    g_ep_probe = &probe;
    const int st = ep_forward_impl((cudaStream_t)stream, comm, cfg, local, x, T, y, workspace, workspace_bytes);
    g_ep_probe = nullptr;
    const cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    for (int i = 0; i < EP_PHASES; ++i) {
        phase_ms[i] = 0.f;
        if (st == CANDLE_MOE_OK && e == cudaSuccess) cudaEventElapsedTime(&phase_ms[i], probe.ev[i], probe.ev[i + 1]);
    }
    if (rows_info) {
        rows_info[0] = probe.rows_received;
        rows_info[1] = probe.rows_busiest_expert;
        EpGeometry g;
        if (st == CANDLE_MOE_OK && e == cudaSuccess && probe.rows_received < 0 && geometry(cfg, local, g) == CANDLE_MOE_OK) {
            // slot form: the counts never left the device during the step; read the table the plan kernel left
            const EpFwdWorkspace ws = fwd_layout(g, local, workspace);
            std::vector<uint32_t> cnt((size_t)g.N * g.El);
            if (cudaMemcpy(cnt.data(), ws.recv_counts, cnt.size() * 4, cudaMemcpyDeviceToHost) == cudaSuccess) {
                int64_t total = 0, busiest = 0;
                for (int le = 0; le < g.El; ++le) {
                    int64_t c = 0;
                    for (int r = 0; r < g.N; ++r) c += cnt[(size_t)r * g.El + le];
                    total += c;
                    busiest = std::max(busiest, c);
                }
                rows_info[0] = total;
                rows_info[1] = busiest;
            }
        }
    }
    for (int i = 0; i <= EP_PHASES; ++i) cudaEventDestroy(probe.ev[i]);
    return st != CANDLE_MOE_OK ? st : rc(e);
}

}  // extern "C"
