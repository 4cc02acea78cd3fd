// Split-KV decode across the GPUs of one box: exchange of the per-head (acc, m, l) partials through
// peer memory and their log-sum-exp merge.
//
// Every rank owns a receive buffer (cudaMalloc) that its peers map (CUDA IPC between processes, peer
// access inside one process).  brc_splitkv_attend / brc_splitkv_step hand the buffers to the decode
// kernel itself (decode_attn.cu): the CTA that completes a (layer, sequence, kv-head group) unit stores
// its merged partial into every rank's buffer and releases a flag per unit, and the CTA that owns the
// unit waits for all ranks' flags at the end of its share and merges - one launch per call, the
// exchange of a layer hidden behind the streaming of the next.  brc_splitkv_exchange_combine is the
// stand-alone second half for a partial the caller already holds: `exchange_merge_kernel`
//   1. stores the partial into its slot of every peer's receive buffer (plain 16-byte global stores
//      over NVLink), fences at system scope, and the CTA that finishes last releases one flag per peer;
//   2. waits, with a time limit, for the flags of all peers in its own buffer, and merges the partials.
// Nothing is pulled from a peer, nothing is multicast, and there is no library collective on the path.
// The reference has no counterpart: its split-K partials never leave one device
// (crates/breccia-kernels/src/qsa/mod.rs:1491-1521).
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#include "../../include/breccia_kv.h"
#include "brc_internal.h"

namespace {

constexpr uint32_t MAX_WORLD = BRC_MAX_WORLD;
constexpr uint32_t N_BANKS = BRC_COMM_BANKS;   // calls in flight between the slowest and the fastest rank: at most 2
constexpr uint32_t FLAG_STRIDE = 32;     // words between flags: one 128-byte line each
constexpr uint64_t DEFAULT_WAIT_NS = 1000000000ull;

struct ExchangeParams {
    uint8_t *peer_recv[MAX_WORLD];   // receive buffers of all ranks as mapped here ([rank] = this rank's own)
    const uint8_t *local_part;       // this rank's partial: acc block then (m, l) block
    uint64_t part_bytes;             // bytes of one partial (multiple of 16)
    uint64_t slot_stride;            // bytes between the slots of two source ranks in a bank
    uint64_t bank_stride;            // bytes between banks
    uint64_t flags_offset;           // byte offset of the flag words in a receive buffer
    uint32_t rank, world;
    uint32_t *calls;                 // local: exchanges completed so far; this call's epoch is that + 1, its bank
                                     // epoch % N_BANKS (kept on the device so that a captured launch replays correctly)
    uint32_t n_rows;                 // n_seqs * n_head
    const float *gate;
    uint32_t gate_head_stride;
    float *out;
    uint32_t *ticket;                // local: CTAs of this launch that finished their stores
    uint32_t *status;                // the pool's check word
    uint64_t wait_ns;
};

__device__ __forceinline__ uint64_t timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ float sigmoid_f32(float x) {
    if (x >= 0.f) return 1.f / (1.f + expf(-x));
    const float e = expf(x);
    return e / (1.f + e);
}

__device__ __forceinline__ uint32_t *flag_of(uint8_t *recv, const ExchangeParams &p, uint32_t bank, uint32_t src) {
    return reinterpret_cast<uint32_t *>(recv + p.flags_offset) + (size_t)(bank * MAX_WORLD + src) * FLAG_STRIDE;
}

// grid <= number of SMs (all CTAs resident: they wait on flags that peers set, never on one another).
template <int HD>
__global__ void __launch_bounds__(HD) exchange_merge_kernel(const ExchangeParams p) {
    __shared__ uint32_t gave_up;
    const uint32_t tid = threadIdx.x;
    if (tid == 0) gave_up = 0;
    // Every CTA reads the call count before it takes its ticket; the last ticket advances it.
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t *>(p.calls) + 1u;
    const uint32_t bank = epoch % N_BANKS;

    // ---- 1. push this rank's partial into its slot at every peer
    {
        const uint64_t n_vec = p.world > 1 ? p.part_bytes / 16 : 0;
        const uint4 *src = reinterpret_cast<const uint4 *>(p.local_part);
        const uint64_t slot = (uint64_t)bank * p.bank_stride + (uint64_t)p.rank * p.slot_stride;
        for (uint64_t i = (uint64_t)blockIdx.x * HD + tid; i < n_vec; i += (uint64_t)gridDim.x * HD) {
            const uint4 v = __ldcg(src + i);
            for (uint32_t r = 0; r < p.world; ++r)
                if (r != p.rank) reinterpret_cast<uint4 *>(p.peer_recv[r] + slot)[i] = v;
        }
        __threadfence_system();
        __syncthreads();
        if (tid == 0) {
            const uint32_t t = atomicAdd(p.ticket, 1u);
            if (t + 1u == gridDim.x) {          // every CTA's stores are fenced: release the flags
                *p.ticket = 0;
                *p.calls = epoch;
                __threadfence_system();
                for (uint32_t r = 0; r < p.world; ++r)
                    if (r != p.rank) st_release_sys(flag_of(p.peer_recv[r], p, bank, p.rank), epoch);
            }
        }
        // ---- 2. wait for every peer's flag in this rank's own buffer (bounded)
        if (tid < p.world && tid != p.rank) {
            const uint32_t *f = flag_of(p.peer_recv[p.rank], p, bank, tid);
            const uint64_t t0 = timer_ns();
            bool ok = false;
            for (uint32_t i = 0; i < (1u << 30); ++i) {
                if ((int32_t)(ld_acquire_sys(f) - epoch) >= 0) { ok = true; break; }
                if ((i & 63u) == 63u && timer_ns() - t0 > p.wait_ns) break;
            }
            if (!ok) {
                gave_up = 1;   // benign race: every writer stores 1
                atomicOr(p.status, BRC_DEV_WAIT_LIMIT);
                p.status[1] = 2000000u + tid;   // which peer never arrived
            }
        }
    }
    __syncthreads();
    if (gave_up) return;   // the call reports a timeout; the output rows are left as they were

    // ---- 3. merge: one row (sequence, head) per CTA pass, one column per thread
    const uint8_t *own = p.peer_recv[p.rank] + (uint64_t)bank * p.bank_stride;
    for (uint32_t row = blockIdx.x; row < p.n_rows; row += gridDim.x) {
        float M = -INFINITY;
        float ms[MAX_WORLD], ls[MAX_WORLD];
#pragma unroll
        for (uint32_t r = 0; r < MAX_WORLD; ++r) {
            if (r < p.world) {
                const uint8_t *part = r == p.rank ? p.local_part : own + (uint64_t)r * p.slot_stride;
                const float2 ml = __ldcg(reinterpret_cast<const float2 *>(part + (size_t)p.n_rows * HD * 4) + row);
                ms[r] = ml.x;
                ls[r] = ml.y;
                if (ml.y > 0.f) M = fmaxf(M, ml.x);
            }
        }
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (uint32_t r = 0; r < MAX_WORLD; ++r) {
            if (r < p.world && ls[r] > 0.f) {
                const uint8_t *part = r == p.rank ? p.local_part : own + (uint64_t)r * p.slot_stride;
                const float w = exp2f(ms[r] - M);
                L += w * ls[r];
                acc += w * __ldcg(reinterpret_cast<const float *>(part) + (size_t)row * HD + tid);
            }
        }
        float v = L > 0.f ? acc / L : 0.f;
        if (p.gate) v *= sigmoid_f32(p.gate[(size_t)row * p.gate_head_stride + tid]);
        p.out[(size_t)row * HD + tid] = v;
    }
}

}  // namespace

struct brc_comm {
    brc_pool *pool = nullptr;
    uint32_t world = 1, rank = 0, max_seqs = 0, n_head = 0;
    uint64_t slot_stride = 0, bank_stride = 0, flags_offset = 0, recv_bytes = 0;
    uint64_t push_offset = 0;          // the banks the decode launch itself stores into (kept full of 0xFF words between exchanges)
    uint32_t unit_items = 0;           // units the buffers hold: max_seqs x kv-head groups
    uint8_t *recv = nullptr;           // this rank's receive buffer (+ flags, + ticket, + local partial)
    uint8_t *local_part = nullptr;     // inside recv's allocation
    uint32_t *ticket = nullptr;        // [0] ticket of the running exchange kernel, [1] exchanges completed, [2] CTAs of the
                                       // running fused launch that have finished
    uint8_t *peer[MAX_WORLD] = {};
    bool opened_ipc[MAX_WORLD] = {};
    bool connected = false;
    uint64_t wait_ns = DEFAULT_WAIT_NS;
};

extern "C" {

brc_status brc_comm_create(brc_pool *pool, uint32_t world, uint32_t rank, uint32_t max_seqs, uint32_t n_head,
                           brc_comm **out) {
    if (!pool || !out) return brc_fail(BRC_ERR_INVALID, "brc_comm_create: NULL pool or result pointer");
    if (pool->device < 0) return brc_fail(BRC_ERR_CUDA, "brc_comm_create: the pool holds bookkeeping only (no device memory)");
    if (world == 0 || world > MAX_WORLD || rank >= world)
        return brc_fail(BRC_ERR_INVALID, "brc_comm_create: rank %u of %u (1 to %u ranks)", rank, world, MAX_WORLD);
    if (max_seqs == 0 || n_head == 0 || n_head % pool->n_kv_head)
        return brc_fail(BRC_ERR_INVALID, "brc_comm_create: %u sequences, %u query heads over %u kv heads", max_seqs, n_head,
                        pool->n_kv_head);
    if (pool->head_dim != 128 && pool->head_dim != 256)
        return brc_fail(BRC_ERR_UNSUPPORTED, "brc_comm_create: head_dim %u (128 or 256)", pool->head_dim);
    brc_device_guard guard(pool->device);
    brc_comm *c = new brc_comm();
    c->pool = pool;
    c->world = world;
    c->rank = rank;
    c->max_seqs = max_seqs;
    c->n_head = n_head;
    uint64_t part = 0;
    brc_decode_partial_bytes(max_seqs, n_head, pool->head_dim, &part);
    c->slot_stride = (part + 255u) & ~255ull;
    c->bank_stride = c->slot_stride * world;
    c->flags_offset = c->bank_stride * N_BANKS;
    const uint64_t flag_bytes = (uint64_t)N_BANKS * MAX_WORLD * FLAG_STRIDE * 4u;
    const uint64_t ticket_off = c->flags_offset + flag_bytes;
    c->unit_items = max_seqs * (pool->n_kv_head / brc_decode_kvb(pool));
    const uint64_t local_off = ticket_off + 256;
    c->push_offset = local_off + c->slot_stride;
    c->recv_bytes = c->push_offset + c->bank_stride * N_BANKS;
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&c->recv), c->recv_bytes);
    if (e != cudaSuccess) {
        delete c;
        return brc_fail(BRC_ERR_CUDA, "brc_comm_create: cudaMalloc of %llu bytes failed: %s", (unsigned long long)c->recv_bytes,
                        cudaGetErrorString(e));
    }
    e = cudaMemset(c->recv, 0, c->recv_bytes);
    if (e != cudaSuccess) {
        cudaFree(c->recv);
        delete c;
        return brc_fail(BRC_ERR_CUDA, "brc_comm_create: cudaMemset failed: %s", cudaGetErrorString(e));
    }
    // the fused exchange has no flags: an empty slot is one that holds 0xFFFFFFFF in every word
    e = cudaMemset(c->recv + c->push_offset, 0xFF, c->bank_stride * N_BANKS);
    if (e != cudaSuccess) {
        cudaFree(c->recv);
        delete c;
        return brc_fail(BRC_ERR_CUDA, "brc_comm_create: cudaMemset failed: %s", cudaGetErrorString(e));
    }
    c->ticket = reinterpret_cast<uint32_t *>(c->recv + ticket_off);
    c->local_part = c->recv + local_off;
    c->peer[rank] = c->recv;
    c->connected = world == 1;
    *out = c;
    return BRC_OK;
}

brc_status brc_comm_ipc_handle(brc_comm *c, void *handle_out64) {
    if (!c || !handle_out64) return brc_fail(BRC_ERR_INVALID, "brc_comm_ipc_handle: NULL argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == BRC_IPC_HANDLE_BYTES, "handle size");
    brc_device_guard guard(c->pool->device);
    cudaIpcMemHandle_t h;
    BRC_CUDA(cudaIpcGetMemHandle(&h, c->recv));
    std::memcpy(handle_out64, &h, sizeof(h));
    return BRC_OK;
}

brc_status brc_comm_connect_ipc(brc_comm *c, const void *handles, uint32_t n_handles) {
    if (!c || !handles) return brc_fail(BRC_ERR_INVALID, "brc_comm_connect_ipc: NULL argument");
    if (n_handles != c->world) return brc_fail(BRC_ERR_INVALID, "brc_comm_connect_ipc: %u handles for %u ranks", n_handles, c->world);
    if (c->connected && c->world > 1) return brc_fail(BRC_ERR_INVALID, "brc_comm_connect_ipc: already connected");
    brc_device_guard guard(c->pool->device);
    for (uint32_t r = 0; r < c->world; ++r) {
        if (r == c->rank) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, static_cast<const uint8_t *>(handles) + (size_t)r * BRC_IPC_HANDLE_BYTES, sizeof(h));
        void *ptr = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess)
            return brc_fail(BRC_ERR_CUDA, "brc_comm_connect_ipc: cannot map the receive buffer of rank %u: %s", r,
                            cudaGetErrorString(e));
        c->peer[r] = static_cast<uint8_t *>(ptr);
        c->opened_ipc[r] = true;
    }
    c->connected = true;
    return BRC_OK;
}

brc_status brc_comm_connect_local(brc_comm *c, brc_comm *const *comms, uint32_t n_comms) {
    if (!c || !comms) return brc_fail(BRC_ERR_INVALID, "brc_comm_connect_local: NULL argument");
    if (n_comms != c->world) return brc_fail(BRC_ERR_INVALID, "brc_comm_connect_local: %u handles for %u ranks", n_comms, c->world);
    brc_device_guard guard(c->pool->device);
    for (uint32_t r = 0; r < c->world; ++r) {
        if (r == c->rank) continue;
        const brc_comm *o = comms[r];
        if (!o || o->world != c->world || o->rank != r || o->slot_stride != c->slot_stride)
            return brc_fail(BRC_ERR_INVALID, "brc_comm_connect_local: entry %u is not rank %u of the same group", r, r);
        if (o->pool->device != c->pool->device) {
            int can = 0;
            BRC_CUDA(cudaDeviceCanAccessPeer(&can, c->pool->device, o->pool->device));
            if (!can)
                return brc_fail(BRC_ERR_UNSUPPORTED, "brc_comm_connect_local: device %d cannot access device %d", c->pool->device,
                                o->pool->device);
            cudaError_t e = cudaDeviceEnablePeerAccess(o->pool->device, 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled)
                cudaGetLastError();
            else if (e != cudaSuccess)
                return brc_fail(BRC_ERR_CUDA, "brc_comm_connect_local: cudaDeviceEnablePeerAccess: %s", cudaGetErrorString(e));
        }
        c->peer[r] = o->recv;
    }
    c->connected = true;
    return BRC_OK;
}

brc_status brc_comm_set_wait_ms(brc_comm *c, uint32_t ms) {
    if (!c || ms == 0) return brc_fail(BRC_ERR_INVALID, "brc_comm_set_wait_ms: NULL handle or zero limit");
    c->wait_ns = (uint64_t)ms * 1000000ull;
    return BRC_OK;
}

brc_status brc_comm_reset(brc_comm *c, void *stream) {
    if (!c) return brc_fail(BRC_ERR_INVALID, "brc_comm_reset: NULL handle");
    brc_device_guard guard(c->pool->device);
    cudaStream_t st = brc_stream(stream);
    BRC_CUDA(cudaMemsetAsync(c->recv + c->push_offset, 0xFF, c->bank_stride * N_BANKS, st));   // every slot empty
    BRC_CUDA(cudaMemsetAsync(c->recv, 0, c->push_offset, st));                                 // flags, tickets, call counts
    BRC_CUDA(cudaStreamSynchronize(st));
    return BRC_OK;
}

brc_status brc_comm_destroy(brc_comm *c) {
    if (!c) return BRC_OK;
    brc_device_guard guard(c->pool->device);
    cudaDeviceSynchronize();
    for (uint32_t r = 0; r < c->world; ++r)
        if (c->opened_ipc[r]) cudaIpcCloseMemHandle(c->peer[r]);
    cudaFree(c->recv);
    delete c;
    return BRC_OK;
}

brc_status brc_splitkv_exchange_combine(brc_comm *c, const void *partial_dev, uint32_t n_seqs, const float *gate_dev,
                                        uint32_t gate_head_stride, float *out_dev, void *stream) {
    if (!c || !out_dev) return brc_fail(BRC_ERR_INVALID, "brc_splitkv_exchange_combine: NULL handle or output");
    if (!c->connected) return brc_fail(BRC_ERR_INVALID, "brc_splitkv_exchange_combine: the peers are not connected yet");
    if (n_seqs > c->max_seqs)
        return brc_fail(BRC_ERR_CAPACITY, "brc_splitkv_exchange_combine: %u sequences but the buffers hold %u", n_seqs, c->max_seqs);
    if (n_seqs == 0) return BRC_OK;
    const uint32_t hd = c->pool->head_dim;
    if (gate_dev && gate_head_stride < hd)
        return brc_fail(BRC_ERR_INVALID, "brc_splitkv_exchange_combine: gate_head_stride %u < head_dim %u", gate_head_stride, hd);
    const uint8_t *part = partial_dev ? static_cast<const uint8_t *>(partial_dev) : c->local_part;
    if (reinterpret_cast<uintptr_t>(part) & 15u)
        return brc_fail(BRC_ERR_INVALID, "brc_splitkv_exchange_combine: the partial must be 16-byte aligned");
    brc_device_guard guard(c->pool->device);
    ExchangeParams p = {};
    for (uint32_t r = 0; r < c->world; ++r) p.peer_recv[r] = c->peer[r];
    p.local_part = part;
    uint64_t bytes = 0;
    brc_decode_partial_bytes(n_seqs, c->n_head, hd, &bytes);
    p.part_bytes = bytes;
    p.slot_stride = c->slot_stride;
    p.bank_stride = c->bank_stride;
    p.flags_offset = c->flags_offset;
    p.calls = c->ticket + 1;
    p.rank = c->rank;
    p.world = c->world;
    p.n_rows = n_seqs * c->n_head;
    p.gate = gate_dev;
    p.gate_head_stride = gate_head_stride;
    p.out = out_dev;
    p.ticket = c->ticket;
    p.status = c->pool->status_dev;
    p.wait_ns = c->wait_ns;
    const uint32_t sms = (uint32_t)(c->pool->sm_count > 0 ? c->pool->sm_count : 148);
    const uint32_t grid = p.n_rows < sms ? p.n_rows : sms;
    cudaStream_t st = brc_stream(stream);
    brc_stage_begin(c->pool, BRC_STAGE_ATTN_COMBINE, st);
    if (hd == 256)
        exchange_merge_kernel<256><<<grid, 256, 0, st>>>(p);
    else
        exchange_merge_kernel<128><<<grid, 128, 0, st>>>(p);
    brc_stage_end(c->pool, BRC_STAGE_ATTN_COMBINE, st);
    BRC_CUDA(cudaGetLastError());
    return BRC_OK;
}

// The comm's buffers as the decode kernel takes them.
static brc_push_args push_args_of(const brc_comm *c) {
    brc_push_args x;
    x.world = c->world;
    x.rank = c->rank;
    for (uint32_t r = 0; r < c->world; ++r) x.peer_recv[r] = c->peer[r];
    x.slot_stride = c->slot_stride;
    x.bank_stride = c->bank_stride;
    x.push_offset = c->push_offset;
    x.unit_items = c->unit_items;
    x.calls = c->ticket + 1;
    x.fin_ticket = c->ticket + 2;
    x.wait_ns = c->wait_ns;
    return x;
}

brc_status brc_splitkv_attend(brc_comm *c, uint32_t layer, const void *q_dev, int32_t q_dtype, const float *gate_dev,
                              uint32_t gate_head_stride, const uint32_t *block_tables_dev, uint32_t table_stride,
                              const uint32_t *seq_lens_dev, uint32_t n_seqs, uint32_t max_seq_len, float scale,
                              float *out_dev, void *workspace_dev, uint64_t workspace_bytes, void *stream) {
    return brc_splitkv_step(c, layer, 1, q_dev, q_dtype, 0, gate_dev, gate_head_stride, block_tables_dev, table_stride, seq_lens_dev,
                            n_seqs, max_seq_len, scale, out_dev, workspace_dev, workspace_bytes, stream);
}

brc_status brc_splitkv_step(brc_comm *c, uint32_t layer0, uint32_t n_layers, const void *q_dev, int32_t q_dtype,
                            uint64_t q_layer_stride_bytes, const float *gate_dev, uint32_t gate_head_stride,
                            const uint32_t *block_tables_dev, uint32_t table_stride, const uint32_t *seq_lens_dev,
                            uint32_t n_seqs, uint32_t max_seq_len, float scale, float *out_dev, void *workspace_dev,
                            uint64_t workspace_bytes, void *stream) {
    const char *who = n_layers == 1 ? "brc_splitkv_attend" : "brc_splitkv_step";
    if (!c) return brc_fail(BRC_ERR_INVALID, "%s: NULL handle", who);
    if (!c->connected) return brc_fail(BRC_ERR_INVALID, "%s: the peers are not connected yet", who);
    if (n_layers == 0 || n_seqs == 0) return BRC_OK;
    if ((uint64_t)n_layers * n_seqs > c->max_seqs)
        return n_layers == 1
                   ? brc_fail(BRC_ERR_CAPACITY, "%s: %u sequences but the buffers hold %u", who, n_seqs, c->max_seqs)
                   : brc_fail(BRC_ERR_CAPACITY, "%s: %u layers x %u sequences but the buffers hold %u (sequence, layer) rows", who,
                              n_layers, n_seqs, c->max_seqs);
    const uint32_t hd = c->pool->head_dim;
    const brc_push_args push = push_args_of(c);
    brc_layers_args a;
    a.layer0 = layer0;
    a.n_layers = n_layers;
    a.q = q_dev;
    a.q_dtype = q_dtype;
    a.q_layer_stride_bytes = q_layer_stride_bytes;
    a.n_head = c->n_head;
    a.gate = gate_dev;
    a.gate_head_stride = gate_head_stride;
    a.gate_layer_stride_bytes = (uint64_t)n_seqs * c->n_head * gate_head_stride * sizeof(float);
    a.block_tables = block_tables_dev;
    a.table_stride = table_stride;
    a.seq_lens = seq_lens_dev;
    a.n_seqs = n_seqs;
    a.max_seq_len = max_seq_len;
    a.scale = scale;
    a.out = out_dev;
    a.out_layer_stride_bytes = (uint64_t)n_seqs * c->n_head * hd * sizeof(float);
    a.workspace = workspace_dev;
    a.workspace_bytes = workspace_bytes;
    a.push = &push;
    return brc_decode_layers(c->pool, who, a, stream);
}

}  // extern "C"
