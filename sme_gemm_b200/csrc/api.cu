// The C ABI (include/smeg_api.h): weight handles, argument checks, kernel
// dispatch, host-pointer wrappers and the drop-in entry points carrying the
// reference's own signatures.  No CPU compute path exists behind any of these:
// a failure returns non-zero and leaves the outputs untouched.
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <chrono>
#include <cmath>
#include <map>
#include <utility>
#include <mutex>
#include <tuple>
#include <vector>

#include "../../include/smeg_api.h"
#include "kernels.h"
#include "layout.h"
#include "handles.h"
#include "pack.h"

using namespace smeg;

// ---------------------------------------------------------------------------
// per-process device state
// ---------------------------------------------------------------------------
namespace {

struct DeviceState {
    bool ok = false;
    int device = -1;
    int sm_count = 0;
    size_t hbm = 0;
    unsigned* status = nullptr;   // device status word (smeg::STATUS_*)
};
std::mutex g_mu;
std::map<int, DeviceState> g_dev;
int g_trace = -1;
// Row count above which the tcgen05 kernel runs instead of the warp-level-MMA decode kernel
// (the reference switches kernels at Linear::PANEL_ROWS = 8 rows, src/linear.rs:160).
// Measured on B200 the decode kernel is faster up to 16 rows.  The tensor-core kernel
// covers every row count; SMEG_TC_MIN_ROWS is a tuning knob.
int g_tc_min_rows = []() {
    const char* e = getenv("SMEG_TC_MIN_ROWS");
    return e ? atoi(e) : 16;
}();

// Rows up to which the decode calls take the direct kernels of gemv_direct.cu (plain loads, packed
// f16 / dp4a arithmetic); 0 keeps them on the ring-staged kernels.  SMEG_DIRECT_ROWS is a tuning knob.
int g_direct_rows = []() {
    const char* e = getenv("SMEG_DIRECT_ROWS");
    const int v = e ? atoi(e) : 4;
    return v < 0 ? 0 : (v > 4 ? 4 : v);
}();

// Rows from which 2-bit / 1-bit calls form their block sums on the tensor cores (lowbit_tc.cu); below it, and above
// the direct kernels' rows, the warp-level kernel runs.  SMEG_LOWBIT_TC_MIN_ROWS is a tuning knob (0 = never).
int g_lowbit_tc = []() {
    const char* e = getenv("SMEG_LOWBIT_TC_MIN_ROWS");
    return e ? atoi(e) : 17;
}();

}  // namespace
// status word of the allocation-free entry point (lowbit_gemv.cu): read and cleared, 0 if never set up
unsigned smeg_static_take_status();
namespace smeg {
bool pdl_enabled() {
    static const bool on = []() {
        const char* e = getenv("SMEG_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}
}  // namespace smeg
namespace {

DeviceState* dev_state() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& s = g_dev[dev];
    if (!s.ok) {
        cudaDeviceProp prop;
        if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return nullptr;
        if (prop.major != 10) {
            fprintf(stderr, "smeg: device %d is sm_%d%d; this library is built for sm_100a only\n", dev, prop.major, prop.minor);
            return nullptr;
        }
        s.device = dev;
        s.sm_count = prop.multiProcessorCount;
        s.hbm = prop.totalGlobalMem;
        if (cudaMalloc(&s.status, sizeof(unsigned)) != cudaSuccess) return nullptr;
        cudaMemset(s.status, 0, sizeof(unsigned));
        // keep freed stream-ordered allocations cached instead of returning them
        cudaMemPool_t pool;
        if (cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
            unsigned long long thr = ~0ull;
            cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &thr);
        }
        s.ok = true;
    }
    return &s;
}

// Scratch of the depth-split tensor-core GEMM (per-slice partial tiles) and of the streaming
// decode kernel (shares of cut column groups plus one arrival counter per column group, zero
// between launches).  One block per (device, stream), so launches that may overlap never share
// it; grown on demand (a synchronous allocation, so the first call of a new size on a stream must
// not be inside a stream capture).  A block that is outgrown is kept until the process ends:
// another host thread may have read its address for a launch it has not issued yet.
struct TcScratch {
    float* ws = nullptr;
    size_t floats = 0;
    int* counters = nullptr;
    size_t ncounters = 0;
};
std::map<std::pair<int, cudaStream_t>, TcScratch> g_tc_scratch;
std::vector<void*> g_retired;        // outgrown blocks, never freed

int tc_scratch(cudaStream_t stream, size_t floats, size_t ncounters, TcScratch* out) {
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lk(g_mu);
    TcScratch& s = g_tc_scratch[{dev, stream}];
    if (s.floats < floats) {
        float* fresh = nullptr;
        if (cudaMalloc(&fresh, floats * sizeof(float)) != cudaSuccess) return -2;
        if (s.ws) g_retired.push_back(s.ws);
        s.ws = fresh;
        s.floats = floats;
    }
    if (s.ncounters < ncounters) {
        int* fresh = nullptr;
        if (cudaMalloc(&fresh, ncounters * sizeof(int)) != cudaSuccess) return -2;
        if (cudaMemset(fresh, 0, ncounters * sizeof(int)) != cudaSuccess) { cudaFree(fresh); return -2; }
        if (s.counters) g_retired.push_back(s.counters);
        s.counters = fresh;
        s.ncounters = ncounters;
    }
    *out = s;
    return 0;
}

// After a kernel gave up on a bounded wait its arrival counters may be left non-zero: clear every
// counter block of the device (the device is idle: the caller has just synchronised it).
void reset_counters_after_timeout(int dev) {
    std::lock_guard<std::mutex> lk(g_mu);
    for (auto& kv : g_tc_scratch)
        if (kv.first.first == dev && kv.second.counters) cudaMemset(kv.second.counters, 0, kv.second.ncounters * sizeof(int));
}

bool tracing() {
    if (g_trace < 0) {
        const char* e = getenv("SMEG_TRACE");
        g_trace = (e && e[0] == '1') ? 1 : 0;
    }
    return g_trace == 1;
}

struct TraceScope {
    const char* name; size_t m, n, k;
    std::chrono::steady_clock::time_point t0;
    bool on;
    TraceScope(const char* nm, size_t m_, size_t n_, size_t k_) : name(nm), m(m_), n(n_), k(k_), on(tracing()) {
        if (on) t0 = std::chrono::steady_clock::now();
    }
    ~TraceScope() {
        if (!on) return;
        const double us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
        fprintf(stderr, "smeg: %s %zux%zux%zu %.1f us\n", name, m, n, k, us);
    }
};

float __uint_as_float_host(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
bool is_pow2(size_t x) { return x != 0 && (x & (x - 1)) == 0; }
bool mul_overflows(size_t a, size_t b) { return a != 0 && b > (size_t)-1 / a; }

template <typename T>
int upload(const std::vector<T>& v, T** out) {
    *out = nullptr;
    const size_t bytes = v.size() * sizeof(T);
    if (cudaMalloc(out, bytes ? bytes : 16) != cudaSuccess) return -2;
    if (bytes && cudaMemcpy(*out, v.data(), bytes, cudaMemcpyHostToDevice) != cudaSuccess) {
        cudaFree(*out);
        *out = nullptr;
        return -2;
    }
    return 0;
}

// Resolve an ep_desc16 into kernel parameters.  With device operand pointers
// (dev = true) nodes are used as they are; `ext_buf` receives a stream-ordered
// device array when the graph is longer than the inline capacity.
int make_ep(const ep_desc16* ep, size_t n, EpParams* out, cudaStream_t stream, EpNodeDev** ext_buf) {
    out->n_nodes = 0;
    out->ext = nullptr;
    *ext_buf = nullptr;
    if (!ep || ep->n_nodes == 0 || !ep->nodes) return 0;
    std::vector<EpNodeDev> nodes(ep->n_nodes);
    for (uint32_t i = 0; i < ep->n_nodes; ++i) {
        const EpNode& s = ep->nodes[i];
        if (s.op > 24u) return -4;
        EpNodeDev d;
        d.op = (s.op & 0xffu) | ((s.aux & 0xffu) << 8);
        d.scalar = s.scalar;
        d.ptr = static_cast<const uint16_t*>(s.ptr);
        d.ld = s.ld == 0 ? n : s.ld;
        nodes[i] = d;
    }
    out->n_nodes = (int)ep->n_nodes;
    if (ep->n_nodes <= (uint32_t)kMaxInlineNodes) {
        for (uint32_t i = 0; i < ep->n_nodes; ++i) out->nodes[i] = nodes[i];
        return 0;
    }
    const size_t bytes = nodes.size() * sizeof(EpNodeDev);
    if (cudaMallocAsync(ext_buf, bytes, stream) != cudaSuccess) return -2;
    if (cudaMemcpyAsync(*ext_buf, nodes.data(), bytes, cudaMemcpyHostToDevice, stream) != cudaSuccess) return -2;
    // pageable source: the copy has been staged by the time the call returns
    out->ext = *ext_buf;
    return 0;
}

bool op_is_row(uint32_t op) { return op == 2 || op == 3 || op == 12 || op == 16 || op == 19 || op == 22; }
bool op_is_col(uint32_t op) { return op == 4 || op == 5 || op == 13 || op == 17 || op == 20 || op == 23; }
bool op_is_tensor(uint32_t op) { return op == 6 || op == 7 || op == 14 || op == 18 || op == 21 || op == 24; }

// Copies a host-pointer op-graph's operands to the device (one allocation) and
// returns a node array with device pointers.  Operand extents follow
// validate_ep (src/exec/guard.rs:112-150): ROW m, COL n, TENSOR (m-1)*ld + n.
struct HostEp {
    std::vector<EpNode> nodes;
    ep_desc16 desc{0, nullptr};
    void* dbuf = nullptr;
    ~HostEp() { if (dbuf) cudaFreeAsync(dbuf, 0); }
    int build(const ep_desc16* ep, size_t m, size_t n) {
        if (!ep || ep->n_nodes == 0 || !ep->nodes) return 0;
        nodes.assign(ep->nodes, ep->nodes + ep->n_nodes);
        size_t total = 0;
        std::vector<size_t> off(nodes.size(), 0), len(nodes.size(), 0);
        for (size_t i = 0; i < nodes.size(); ++i) {
            const EpNode& s = nodes[i];
            size_t l = 0;
            if (op_is_row(s.op)) l = m;
            else if (op_is_col(s.op)) l = n;
            else if (op_is_tensor(s.op)) {
                const size_t ld = s.ld == 0 ? n : s.ld;
                if (ld < n) return -4;
                l = m == 0 ? 0 : (m - 1) * ld + n;
            }
            if (l && !s.ptr) return -4;
            len[i] = l;
            off[i] = total;
            total += (l * 2 + 15) / 16 * 16;
        }
        if (total) {
            if (cudaMallocAsync(&dbuf, total, 0) != cudaSuccess) return -2;   // (cached by the pool: no synchronising allocation per call)
            for (size_t i = 0; i < nodes.size(); ++i)
                if (len[i]) {
                    if (cudaMemcpy((char*)dbuf + off[i], nodes[i].ptr, len[i] * 2, cudaMemcpyHostToDevice) != cudaSuccess) return -2;
                    nodes[i].ptr = (char*)dbuf + off[i];
                }
        }
        desc.n_nodes = (uint32_t)nodes.size();
        desc.nodes = nodes.data();
        return 0;
    }
    const ep_desc16* get() const { return desc.n_nodes ? &desc : nullptr; }
};

}  // namespace

// ---------------------------------------------------------------------------
// handles
// ---------------------------------------------------------------------------
extern "C" {

const char* smeg_version(void) { return "sme-gemm-b200 0.1 (sm_100a)"; }

int smeg_device_info(int* sm_count, size_t* hbm_bytes) {
    DeviceState* s = dev_state();
    if (!s) return -5;
    if (sm_count) *sm_count = s->sm_count;
    if (hbm_bytes) *hbm_bytes = s->hbm;
    return 0;
}

unsigned smeg_last_status(void) {
    DeviceState* s = dev_state();
    if (!s) return ~0u;
    unsigned v = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return ~0u;
    cudaMemcpy(&v, s->status, sizeof(v), cudaMemcpyDeviceToHost);
    if (v) cudaMemset(s->status, 0, sizeof(unsigned));
    v |= smeg_static_take_status();
    if (v) reset_counters_after_timeout(s->device);
    return v;
}

void smeg_trace(int on) { g_trace = on ? 1 : 0; }

// ---- Q4 handles ----
// An affine handle keeps the logical arrays; its dense twins are built by q4_affine_twin on first use.
static int q4_finish_affine(std::vector<uint8_t>& quants, std::vector<uint16_t>& scales, std::vector<uint16_t>& mins, size_t n, size_t k,
                            size_t block, smeg_q4** out) {
    if (!dev_state()) return -5;
    smeg_q4* h = new smeg_q4();
    h->d = make_dims(n, k, block, kQ4UnitDepth);
    h->affine = true;
    h->h_quants.swap(quants);
    h->h_scales.swap(scales);
    h->h_mins.swap(mins);
    *out = h;
    return 0;
}

static int q4_finish(const std::vector<uint8_t>& quants, const std::vector<uint16_t>& scales, size_t n, size_t k,
                     size_t block, smeg_q4** out) {
    if (!dev_state()) return -5;
    smeg_q4* h = new smeg_q4();
    h->d = make_dims(n, k, block, kQ4UnitDepth);
    std::vector<uint8_t> codes;
    std::vector<uint16_t> sc;
    q4_pack(quants.data(), scales.data(), h->d, codes, sc);
    h->code_bytes = codes.size();
    h->scale_elems = sc.size();
    if (upload(codes, &h->codes) || upload(sc, &h->scales)) {
        smeg_q4_destroy(h);
        return -2;
    }
    *out = h;
    return 0;
}

int smeg_q4_create(const uint8_t* quants, const uint16_t* scales, const uint16_t* mins, size_t n, size_t k,
                   size_t block, smeg_q4** out) {
    if (!out) return -4;
    *out = nullptr;
    if (!is_pow2(block)) return -1;
    if (mul_overflows(n, k) || ((n != 0 && k != 0) && (!quants || !scales))) return -4;
    const size_t nbk = div_up(k, block);
    std::vector<uint8_t> q(quants, quants + (n * k + 1) / 2);
    std::vector<uint16_t> s(scales, scales + n * nbk);
    if (mins) {
        std::vector<uint16_t> mn(mins, mins + n * nbk);
        return q4_finish_affine(q, s, mn, n, k, block, out);
    }
    return q4_finish(q, s, n, k, block, out);
}

int smeg_q4_quantize(const float* w, int layout, size_t n, size_t k, size_t block, int affine, smeg_q4** out) {
    if (!out) return -4;
    *out = nullptr;
    if (!is_pow2(block)) return -1;
    if (mul_overflows(n, k) || ((n != 0 && k != 0) && !w)) return -4;
    std::vector<uint8_t> q;
    std::vector<uint16_t> s, mn;
    q4_quantize_host(w, layout, n, k, block, affine ? 1 : 0, q, s, mn);
    if (affine) return q4_finish_affine(q, s, mn, n, k, block, out);
    return q4_finish(q, s, n, k, block, out);
}

int smeg_q4_from_band(const uint8_t* nibbles, const uint16_t* scales, const uint16_t* mins, size_t n, size_t k,
                      size_t block, smeg_q4** out) {
    if (!out) return -4;
    *out = nullptr;
    if (!is_pow2(block)) return -1;
    if (mul_overflows(n, k) || ((n != 0 && k != 0) && (!nibbles || !scales))) return -4;
    std::vector<uint8_t> q;
    std::vector<uint16_t> s, mn;
    q4_from_band(nibbles, scales, mins, n, k, block, q, s, mn);
    if (mins) return q4_finish_affine(q, s, mn, n, k, block, out);
    return q4_finish(q, s, n, k, block, out);
}

void smeg_q4_destroy(smeg_q4* w) {
    if (!w) return;
    if (smeg_dense* t = w->twin_f16.load()) smeg_dense_destroy(t);
    if (smeg_dense* t = w->twin_bf16.load()) smeg_dense_destroy(t);
    if (w->codes) cudaFree(w->codes);
    if (w->scales) cudaFree(w->scales);
    delete w;
}
size_t smeg_q4_n(const smeg_q4* w) { return w->d.n; }
size_t smeg_q4_k(const smeg_q4* w) { return w->d.k; }
size_t smeg_q4_block(const smeg_q4* w) { return w->d.block; }
size_t smeg_q4_device_bytes(const smeg_q4* w) {
    if (w->affine) return ((w->twin_f16.load() ? 1 : 0) + (w->twin_bf16.load() ? 1 : 0)) * w->d.n * ((w->d.k + 7) / 8 * 8) * 2;
    return w->code_bytes + w->scale_elems * 2;
}

int smeg_q4_unpack(const smeg_q4* w, uint8_t* quants, uint16_t* scales) {
    if (!w || !quants || !scales) return -4;
    if (w->affine) {
        memcpy(quants, w->h_quants.data(), w->h_quants.size());
        memcpy(scales, w->h_scales.data(), w->h_scales.size() * 2);
        return 0;
    }
    std::vector<uint8_t> codes(w->code_bytes);
    std::vector<uint16_t> sc(w->scale_elems);
    if (w->code_bytes && cudaMemcpy(codes.data(), w->codes, w->code_bytes, cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
    if (w->scale_elems && cudaMemcpy(sc.data(), w->scales, w->scale_elems * 2, cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
    q4_unpack(codes.data(), sc.data(), w->d, quants, scales);
    return 0;
}

// ---- 2-bit / 1-bit handles ----
static int lowbit_finish(int bits, const uint8_t* wbits, int layout, const uint16_t* scales, size_t n, size_t k,
                         size_t block, const int8_t* codebook, smeg_lowbit** out) {
    if (!dev_state()) return -5;
    smeg_lowbit* h = new smeg_lowbit();
    h->bits = bits;
    h->d = make_dims(n, k, block, bits == 2 ? kQ2UnitDepth : kQ1UnitDepth);
    if (codebook) {
        memcpy(h->codebook, codebook, 4);
        h->lut = (uint32_t)(uint8_t)codebook[0] | ((uint32_t)(uint8_t)codebook[1] << 8) |
                 ((uint32_t)(uint8_t)codebook[2] << 16) | ((uint32_t)(uint8_t)codebook[3] << 24);
    }
    std::vector<uint8_t> codes;
    std::vector<uint16_t> sc;
    if (bits == 2) q2_pack(wbits, scales, h->d, codes, sc);
    else q1_pack(wbits, layout, scales, h->d, codes, sc);
    h->code_bytes = codes.size();
    h->scale_elems = sc.size();
    if (upload(codes, &h->codes) || upload(sc, &h->scales)) {
        smeg_lowbit_destroy(h);
        return -2;
    }
    *out = h;
    return 0;
}
static bool lowbit_block_ok(size_t block) { return is_pow2(block) && block >= 16 && block <= 65536; }

int smeg_q2_create(const uint8_t* codes, const uint16_t* scales, size_t n, size_t k, size_t block,
                   const int8_t codebook[4], smeg_lowbit** out) {
    if (!out || !codebook) return -4;
    *out = nullptr;
    if (!lowbit_block_ok(block)) return -1;
    if (mul_overflows(n, k) || ((n != 0 && k != 0) && (!codes || !scales))) return -4;
    return lowbit_finish(2, codes, 1, scales, n, k, block, codebook, out);
}
int smeg_q2_quantize(const float* w, int layout, size_t n, size_t k, size_t block, const int8_t codebook[4],
                     smeg_lowbit** out) {
    if (!out || !codebook) return -4;
    *out = nullptr;
    if (!lowbit_block_ok(block)) return -1;
    if (mul_overflows(n, k) || ((n != 0 && k != 0) && !w)) return -4;
    std::vector<uint8_t> codes;
    std::vector<uint16_t> sc;
    if (q2_quantize_host(w, layout, n, k, block, codebook, codes, sc)) return -2;
    return lowbit_finish(2, codes.data(), 1, sc.data(), n, k, block, codebook, out);
}
int smeg_q1_create(const uint8_t* signs, const uint16_t* scales, int layout, size_t n, size_t k, size_t block,
                   smeg_lowbit** out) {
    if (!out) return -4;
    *out = nullptr;
    if (!lowbit_block_ok(block)) return -1;
    if (mul_overflows(n, k) || ((n != 0 && k != 0) && (!signs || !scales))) return -4;
    return lowbit_finish(1, signs, layout, scales, n, k, block, nullptr, out);
}
int smeg_q1_quantize(const float* w, int layout, size_t n, size_t k, size_t block, smeg_lowbit** out) {
    if (!out) return -4;
    *out = nullptr;
    if (!lowbit_block_ok(block)) return -1;
    if (mul_overflows(n, k) || ((n != 0 && k != 0) && !w)) return -4;
    std::vector<uint8_t> signs;
    std::vector<uint16_t> sc;
    q1_quantize_host(w, layout, n, k, block, signs, sc);
    return lowbit_finish(1, signs.data(), 0, sc.data(), n, k, block, nullptr, out);
}
int smeg_q2_from_band(const uint8_t* codes, const uint16_t* scales, size_t n, size_t k, size_t block,
                      const int8_t codebook[4], smeg_lowbit** out) {
    if (!out || !codebook) return -4;
    *out = nullptr;
    if (!lowbit_block_ok(block)) return -1;
    if (mul_overflows(n, k) || ((n != 0 && k != 0) && (!codes || !scales))) return -4;
    std::vector<uint8_t> c;
    std::vector<uint16_t> s;
    q2_from_band(codes, scales, n, k, block, c, s);
    return lowbit_finish(2, c.data(), 1, s.data(), n, k, block, codebook, out);
}
int smeg_q1_from_band(const uint8_t* signs, const uint16_t* scales, size_t n, size_t k, size_t block,
                      smeg_lowbit** out) {
    if (!out) return -4;
    *out = nullptr;
    if (!lowbit_block_ok(block)) return -1;
    if (mul_overflows(n, k) || ((n != 0 && k != 0) && (!signs || !scales))) return -4;
    std::vector<uint8_t> c;
    std::vector<uint16_t> s;
    q1_from_band(signs, scales, n, k, block, c, s);
    return lowbit_finish(1, c.data(), 0, s.data(), n, k, block, nullptr, out);
}
void smeg_lowbit_destroy(smeg_lowbit* w) {
    if (!w) return;
    smeg_q4_destroy(w->twin.load());
    smeg_dense_destroy(w->twin_dense.load());
    if (w->codes) cudaFree(w->codes);
    if (w->scales) cudaFree(w->scales);
    delete w;
}
size_t smeg_lowbit_n(const smeg_lowbit* w) { return w->d.n; }
size_t smeg_lowbit_k(const smeg_lowbit* w) { return w->d.k; }
size_t smeg_lowbit_block(const smeg_lowbit* w) { return w->d.block; }
int smeg_lowbit_bits(const smeg_lowbit* w) { return w->bits; }
size_t smeg_lowbit_device_bytes(const smeg_lowbit* w) { return w->code_bytes + w->scale_elems * 2; }
int smeg_lowbit_unpack(const smeg_lowbit* w, uint8_t* bits_out, uint16_t* scales) {
    if (!w || !bits_out || !scales) return -4;
    std::vector<uint8_t> codes(w->code_bytes);
    std::vector<uint16_t> sc(w->scale_elems);
    if (w->code_bytes && cudaMemcpy(codes.data(), w->codes, w->code_bytes, cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
    if (w->scale_elems && cudaMemcpy(sc.data(), w->scales, w->scale_elems * 2, cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
    if (w->bits == 2) q2_unpack(codes.data(), sc.data(), w->d, bits_out, scales);
    else q1_unpack(codes.data(), sc.data(), w->d, bits_out, scales);
    return 0;
}

// ---- host-side preparation on caller buffers (no device) ----
static int unit_depth_of(int bits) { return bits == 4 ? kQ4UnitDepth : (bits == 2 ? kQ2UnitDepth : (bits == 1 ? kQ1UnitDepth : 0)); }

size_t smeg_packed_code_bytes(int bits, size_t n, size_t k) {
    const int ud = unit_depth_of(bits);
    if (!ud) return 0;
    const PackedDims d = make_dims(n, k, 32, ud);
    return d.n16 * d.ku * kUnitBytes;
}
size_t smeg_packed_scale_elems(int bits, size_t n, size_t k, size_t block) {
    const int ud = unit_depth_of(bits);
    if (!ud || !is_pow2(block)) return 0;
    const PackedDims d = make_dims(n, k, block, ud);
    return d.n16 * d.nb * 16;
}
int smeg_host_pack(int bits, const uint8_t* wbits, int layout, const uint16_t* scales, size_t n, size_t k,
                   size_t block, uint8_t* codes_out, uint16_t* scales_out) {
    const int ud = unit_depth_of(bits);
    if (!ud || !is_pow2(block) || mul_overflows(n, k)) return -4;
    const PackedDims d = make_dims(n, k, block, ud);
    std::vector<uint8_t> codes;
    std::vector<uint16_t> sc;
    if (bits == 4) q4_pack(wbits, scales, d, codes, sc);
    else if (bits == 2) q2_pack(wbits, scales, d, codes, sc);
    else q1_pack(wbits, layout, scales, d, codes, sc);
    if (!codes.empty()) memcpy(codes_out, codes.data(), codes.size());
    if (!sc.empty()) memcpy(scales_out, sc.data(), sc.size() * 2);
    return 0;
}
int smeg_host_unpack(int bits, const uint8_t* codes, const uint16_t* packed_scales, size_t n, size_t k,
                     size_t block, uint8_t* wbits_out, uint16_t* scales_out) {
    const int ud = unit_depth_of(bits);
    if (!ud || !is_pow2(block) || mul_overflows(n, k)) return -4;
    const PackedDims d = make_dims(n, k, block, ud);
    if (bits == 4) q4_unpack(codes, packed_scales, d, wbits_out, scales_out);
    else if (bits == 2) q2_unpack(codes, packed_scales, d, wbits_out, scales_out);
    else q1_unpack(codes, packed_scales, d, wbits_out, scales_out);
    return 0;
}
int smeg_host_q4_quantize(const float* w, int layout, size_t n, size_t k, size_t block, uint8_t* quants,
                          uint16_t* scales) {
    if (!is_pow2(block)) return -1;
    if (mul_overflows(n, k)) return -4;
    std::vector<uint8_t> q;
    std::vector<uint16_t> s, mn;
    q4_quantize_host(w, layout, n, k, block, 0, q, s, mn);
    if (!q.empty()) memcpy(quants, q.data(), q.size());
    if (!s.empty()) memcpy(scales, s.data(), s.size() * 2);
    return 0;
}
int smeg_host_q2_quantize(const float* w, int layout, size_t n, size_t k, size_t block, const int8_t codebook[4],
                          uint8_t* codes, uint16_t* scales) {
    if (!lowbit_block_ok(block)) return -1;
    if (mul_overflows(n, k) || !codebook) return -4;
    std::vector<uint8_t> c;
    std::vector<uint16_t> s;
    if (q2_quantize_host(w, layout, n, k, block, codebook, c, s)) return -2;
    if (!c.empty()) memcpy(codes, c.data(), c.size());
    if (!s.empty()) memcpy(scales, s.data(), s.size() * 2);
    return 0;
}
int smeg_host_q1_quantize(const float* w, int layout, size_t n, size_t k, size_t block, uint8_t* signs,
                          uint16_t* scales) {
    if (!lowbit_block_ok(block)) return -1;
    if (mul_overflows(n, k)) return -4;
    std::vector<uint8_t> sg;
    std::vector<uint16_t> s;
    q1_quantize_host(w, layout, n, k, block, sg, s);
    if (!sg.empty()) memcpy(signs, sg.data(), sg.size());
    if (!s.empty()) memcpy(scales, s.data(), s.size() * 2);
    return 0;
}

// ---------------------------------------------------------------------------
// device-pointer compute
// ---------------------------------------------------------------------------
// Whether an m-row call on these weights runs on the tensor-core GEMM (else the decode kernel).
static bool q4_uses_tc(const smeg_q4* w, const uint16_t* a, size_t m) {
    return (int)m > g_tc_min_rows && gemm_tc_supported(4, (int)m, (int)w->d.k, w->d.log2_block, a);
}

static float half_bits_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, ex = (h >> 10) & 0x1fu, man = h & 0x3ffu;
    float f;
    if (ex == 0) {
        f = std::ldexp((float)man, -24);
        return sign ? -f : f;
    }
    const uint32_t bits = ex == 31 ? (sign | 0x7f800000u | (man << 13)) : (sign | ((ex + 112u) << 23) | (man << 13));
    memcpy(&f, &bits, 4);
    return f;
}
// f64 -> f16 bits, round to nearest even, one rounding (the values here are far from overflow; handled all the same).
static uint16_t f64_to_f16_bits(double v) {
    if (v != v) return 0x7e00;
    const uint16_t sign = std::signbit(v) ? 0x8000 : 0;
    const double a = std::fabs(v);
    if (a >= 65520.0) return sign | 0x7c00;
    if (a < 6.103515625e-05) return sign | (uint16_t)std::nearbyint(a * 16777216.0);   // subnormal: quantum 2^-24
    int e;
    (void)std::frexp(a, &e);
    int m10 = (int)std::nearbyint((std::ldexp(a, 1 - e) - 1.0) * 1024.0), ex = e - 1 + 15;
    if (m10 == 1024) { m10 = 0; ++ex; }
    if (ex >= 31) return sign | 0x7c00;
    return sign | (uint16_t)(ex << 10) | (uint16_t)m10;
}
static uint16_t f32_to_bf16_bits(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40);
    return (uint16_t)((x + 0x7fffu + ((x >> 16) & 1u)) >> 16);
}

// The dense twin of an affine handle for one operand type: W[n][kd] = round_T(f64(scale) * code + f64(min)), T = f16
// straight from f64, bf16 through f32 (dequant_rows, src/kernels/q4/weights.rs:232-259).
static int q4_affine_twin(const smeg_q4* w, int bf16, const smeg_dense** out) {
    std::atomic<smeg_dense*>& slot = bf16 ? w->twin_bf16 : w->twin_f16;
    smeg_dense* t = slot.load(std::memory_order_acquire);
    if (t) { *out = t; return 0; }
    std::lock_guard<std::mutex> lock(w->twin_lock);
    t = slot.load(std::memory_order_acquire);
    if (t) { *out = t; return 0; }
    const size_t n = w->d.n, k = w->d.k, block = w->d.block, nbk = div_up(k, block), kd = (k + 7) / 8 * 8;
    std::vector<uint16_t> dense(n * kd, 0);
    for (size_t d = 0; d < k; ++d)
        for (size_t j = 0; j < n; ++j) {
            const size_t idx = d * n + j;
            const int nib = (idx % 2 == 0) ? (w->h_quants[idx / 2] & 0x0f) : (w->h_quants[idx / 2] >> 4);
            const int code = nib < 8 ? nib : nib - 16;
            const size_t si = j * nbk + d / block;
            const double v = (double)half_bits_to_float(w->h_scales[si]) * (double)code + (double)half_bits_to_float(w->h_mins[si]);
            dense[j * kd + d] = bf16 ? f32_to_bf16_bits((float)v) : f64_to_f16_bits(v);
        }
    smeg_dense* h = new smeg_dense();
    h->n = n; h->k = k; h->kd = kd; h->bf16 = bf16 ? 1 : 0;
    if (upload(dense, &h->w)) { smeg_dense_destroy(h); return -2; }
    slot.store(h, std::memory_order_release);
    *out = h;
    return 0;
}

// Does a call of m rows run on the one-wave decode kernel (gemv_direct.cu)?  With glu: also that the matrix interleaves
// whole 32-column gate / up chunks.
static bool q4_takes_direct(const smeg_q4* w, const uint16_t* a, size_t m, int bf16, int glu) {
    if (w->affine || q4_uses_tc(w, a, m) || g_direct_rows <= 0 || (int)m > g_direct_rows) return false;
    if (glu && w->d.n % 64 != 0) return false;
    Q4GemvArgs g;
    memset(&g, 0, sizeof(g));
    g.m = (int)m; g.n = (int)w->d.n; g.k = (int)w->d.k; g.k64 = (int)w->d.ku; g.log2_block = w->d.log2_block;
    g.a_vec_ok = (w->d.k % 8 == 0) && ((uintptr_t)a % 16 == 0);
    return q4_direct_supported(g, bf16);
}

// glu / yacc: the fused forms of the MLP block (the tensor-core GEMM, and the one-wave decode kernel at up to four rows).
struct TpPush { float* bufs[8]; int world, rank, rows; };
static int q4_dev(const smeg_q4* w, const uint16_t* a, uint16_t* c, size_t m, const ep_desc16* ep, int bf16,
                  cudaStream_t stream, float* c32 = nullptr, int glu = 0, float* yacc = nullptr, const TpPush* push = nullptr) {
    if (!w) return -4;
    const size_t n = w->d.n, k = w->d.k;
    if (m == 0 || n == 0) return 0;
    if ((!c && !c32 && !yacc) || (k && !a) || m > 0x7fffffffu || n > 0x7fffffffu || k > 0x7fffffffu) return -4;
    if (w->affine) {
        if (c32 || glu || yacc) return -3;                       // the fused forms of the MLP block take Q4_0 weights
        const smeg_dense* t = nullptr;
        const int rc = q4_affine_twin(w, bf16, &t);
        if (rc) return rc;
        return smeg_gemm_dense_dev(t, a, c, m, bf16 ? 0x3f80 : 0x3c00 /* beta = 1 */, 0, ep, stream);
    }
    if ((glu || yacc) && !q4_uses_tc(w, a, m) && !q4_takes_direct(w, a, m, bf16, glu)) return -4;
    if (push && (!c32 || !q4_uses_tc(w, a, m))) return -3;
    DeviceState* ds = dev_state();
    if (!ds) return -5;
    Q4GemvArgs g;
    memset(&g, 0, sizeof(g));
    EpNodeDev* ext = nullptr;
    int rc = make_ep(ep, n, &g.ep, stream, &ext);
    if (rc) { if (ext) cudaFreeAsync(ext, stream); return rc; }
    g.codes = w->codes; g.scales = w->scales; g.a = a; g.c = c; g.c32 = c32;
    g.m = (int)m; g.n = (int)n; g.k = (int)k;
    g.n16 = (int)w->d.n16; g.k64 = (int)w->d.ku; g.nb = (int)w->d.nb;
    g.log2_block = w->d.log2_block;
    g.a_vec_ok = (k % 8 == 0) && ((uintptr_t)a % 16 == 0);
    g.status = ds->status;
    cudaError_t e;
    if (q4_uses_tc(w, a, m)) {
        GemmTcArgs t;
        memset(&t, 0, sizeof(t));
        t.codes = w->codes; t.scales = w->scales; t.a = a; t.c = c; t.c32 = c32; t.glu = glu; t.yacc = yacc;
        t.m = (int)m; t.n = (int)n; t.k = (int)k;
        t.n16 = (int)w->d.n16; t.ku = (int)w->d.ku; t.nb = (int)w->d.nb; t.log2_block = w->d.log2_block;
        t.status = ds->status;
        t.ep = g.ep;
        if (push) {
            for (int s = 0; s < push->world; ++s) t.push[s] = push->bufs[s];
            t.push_world = push->world; t.push_rank = push->rank; t.push_rows = push->rows;
        }
        dim3 grid;
        size_t smem = 0, ws_floats = 0, ncounters = 0;
        gemm_tc_plan(t, ds->sm_count, &grid, &smem, &ws_floats, &ncounters);
        TcScratch sc;
        if (ws_floats && tc_scratch(stream, ws_floats, ncounters, &sc)) {
            if (ext) cudaFreeAsync(ext, stream);
            return -2;
        }
        t.ws = sc.ws;
        t.counters = sc.counters;
        e = gemm_tc_launch(t, bf16, grid, smem, stream);
    } else if (g_direct_rows > 0 && (int)m <= g_direct_rows && q4_direct_supported(g, bf16)) {
        g.glu = glu; g.yacc = yacc;
        e = q4_direct_launch(g, ds->sm_count, stream);
    } else {
        size_t ws_floats = 0, ncounters = 0;
        q4_gemv_stream_plan(g, bf16, ds->sm_count, &ws_floats, &ncounters);
        if (g.sgrid) {
            TcScratch sc;
            if (tc_scratch(stream, ws_floats, ncounters, &sc)) {
                if (ext) cudaFreeAsync(ext, stream);
                return -2;
            }
            g.ws = sc.ws;
            g.counters = sc.counters;
        }
        e = q4_gemv_launch(g, bf16, ds->sm_count, stream);
    }
    if (ext) cudaFreeAsync(ext, stream);
    return e == cudaSuccess ? 0 : -6;
}

int smeg_matmul_q4_f16_dev(const smeg_q4* w, const uint16_t* a, uint16_t* c, size_t m, const ep_desc16* ep, void* stream) {
    return q4_dev(w, a, c, m, ep, 0, (cudaStream_t)stream);
}
int smeg_matmul_q4_bf16_dev(const smeg_q4* w, const uint16_t* a, uint16_t* c, size_t m, const ep_desc16* ep, void* stream) {
    return q4_dev(w, a, c, m, ep, 1, (cudaStream_t)stream);
}
int smeg_matmul_q4_partial_dev(const smeg_q4* w, const uint16_t* a, float* partial, size_t m, void* stream) {
    if (!partial) return -4;
    return q4_dev(w, a, nullptr, m, nullptr, 0, (cudaStream_t)stream, partial);
}

static int lowbit_dev(const smeg_lowbit* w, const uint16_t* a, uint16_t* c, size_t m, const ep_desc16* ep,
                      int8_t* q_out, float* sa_out, int32_t* sums_out, cudaStream_t stream) {
    if (!w) return -4;
    const size_t n = w->d.n, k = w->d.k;
    if (m == 0 || n == 0) return 0;
    if (!c || (k && !a) || m > 0x7fffffffu || n > 0x7fffffffu || k > 0x7fffffffu) return -4;
    DeviceState* ds = dev_state();
    if (!ds) return -5;
    const size_t kq = w->d.ku * (size_t)w->d.unit_depth, nb = w->d.nb;
    LowbitGemvArgs g;
    memset(&g, 0, sizeof(g));
    EpNodeDev* ext = nullptr;
    int rc = make_ep(ep, n, &g.ep, stream, &ext);
    if (rc) { if (ext) cudaFreeAsync(ext, stream); return rc; }
    g.codes = w->codes; g.scales = w->scales; g.c = c;
    g.sums_out = sums_out;
    g.m = (int)m; g.n = (int)n; g.k = (int)k; g.kq = (int)kq;
    g.n16 = (int)w->d.n16; g.ku = (int)w->d.ku; g.nb = (int)nb; g.nb_real = (int)w->d.nb_real;
    g.log2_block = w->d.log2_block; g.lut = w->lut; g.status = ds->status;
    cudaError_t e = cudaSuccess;
    char* ws = nullptr;
    // up to four rows the kernel stages and quantises the activations itself (one launch, no scratch);
    // above that every CTA would repeat too much work, and a separate pass over the rows is faster
    static const size_t fuse_max_rows = []() { const char* e = getenv("SMEG_LB_FUSE_MAX_ROWS"); return e ? (size_t)atoi(e) : (size_t)4; }();
    g.a_vec_ok = (k % 8 == 0) && ((uintptr_t)a % 16 == 0);
    if (k > 0 && (int)m <= g_direct_rows && m <= 2 && (g.a = a, lowbit_direct_supported(g, true))) {
        // one or two rows: the direct kernel quantises the rows itself in every CTA
        g.q_out = q_out; g.sa_out = sa_out;
        e = lowbit_direct_launch(g, w->bits, ds->sm_count, stream);
    } else if (g.a = nullptr, k > 0 && g_direct_rows == 0 && m <= fuse_max_rows && (k % 8 == 0) && ((uintptr_t)a % 16 == 0) && lowbit_gemv_fuses_quant(g, w->bits, ds->sm_count)) {
        // the kernel quantises the activation rows itself: one launch, no scratch
        g.a = a;
        g.a_vec_ok = 1;
        g.q_out = q_out; g.sa_out = sa_out;
        e = lowbit_gemv_launch(g, w->bits, ds->sm_count, stream);
    } else {
        // quantise first, into stream-ordered scratch; above the direct kernels' rows the block sums run on the
        // tensor cores (lowbit_tc.cu), which wants the per-block scales and sums block-major as well
        const bool tc = (int)m > g_direct_rows && g_lowbit_tc > 0 && (int)m >= g_lowbit_tc && lowbit_tc_supported(w->bits, (int)m, (int)k, w->d.log2_block);
        // between the two, warp-level tensor-core instructions (lowbit_mma.cu); SMEG_LOWBIT_MMA=0 leaves those row counts
        // to the staged dp4a kernel
        static const int use_mma = []() { const char* e = getenv("SMEG_LOWBIT_MMA"); return e ? atoi(e) : 1; }();
        bool mma = false;
        if (!tc && use_mma && (int)m > g_direct_rows && m <= 16) {
            LowbitGemvArgs probe = g;
            probe.qh = (const uint16_t*)1; probe.sa = (const float*)1; probe.qsum = (const int32_t*)1;   // set below
            mma = lowbit_mma_supported(probe, ds->sm_count);
        }
        const size_t mpad = (m + 127) / 128 * 128;                     // whole row tiles of the tensor-core kernel (up to 128 rows)
        const size_t q_bytes = (m * kq + 255) / 256 * 256, sa_bytes = (m * nb * 4 + 255) / 256 * 256;
        const size_t t_bytes = tc ? (mpad * nb * 4 + 255) / 256 * 256 : 0, qh_bytes = (tc || mma) ? ((m + 7) / 8 * 8 * kq * 2 + 255) / 256 * 256 : 0;
        if (cudaMallocAsync(&ws, q_bytes + 2 * sa_bytes + 2 * t_bytes + qh_bytes + 256, stream) != cudaSuccess) {
            if (ext) cudaFreeAsync(ext, stream);
            return -2;
        }
        ActQuantArgs aq;
        memset(&aq, 0, sizeof(aq));
        aq.a = a; aq.q = (int8_t*)ws; aq.sa = (float*)(ws + q_bytes);
        aq.qsum = (w->bits == 1 || tc || mma) ? (int32_t*)(ws + q_bytes + sa_bytes) : nullptr;
        aq.m = (int)m; aq.k = (int)k; aq.kq = (int)kq; aq.nbq = (int)nb; aq.log2_block = w->d.log2_block;
        if (tc) {
            aq.sa_t = (float*)(ws + q_bytes + 2 * sa_bytes);
            aq.qsum_t = (float*)(ws + q_bytes + 2 * sa_bytes + t_bytes);
            aq.qh = (uint16_t*)(ws + q_bytes + 2 * sa_bytes + 2 * t_bytes);
            aq.mpad = (int)mpad;
            aq.qh_perm = w->bits == 1 ? 2 : 0;                         // 1-bit: the order and scaling the kernel's operand tiles take
        }
        if (mma) {
            aq.qh = (uint16_t*)(ws + q_bytes + 2 * sa_bytes + 2 * t_bytes);
            aq.qh_perm = w->bits == 1 ? 2 : 0;                         // 1-bit: fragment order, codes scaled by position
            // the rows up to the next multiple of eight are zero rows (the kernel's B fragments read whole tiles of eight)
            if (m % 8 != 0) cudaMemsetAsync(aq.qh + m * kq, 0, (8 - m % 8) * kq * 2, stream);
        }
        e = act_quant_launch(aq, stream);
        g.q = aq.q; g.sa = aq.sa; g.qsum = aq.qsum; g.qh = aq.qh;
        if (e == cudaSuccess) {
            if (tc) {
                LowbitTcArgs t;
                memset(&t, 0, sizeof(t));
                t.codes = w->codes; t.scales = w->scales; t.qh = aq.qh; t.sa_t = aq.sa_t; t.qsum_t = aq.qsum_t; t.mpad = (int)mpad;
                t.c = c; t.sums_out = sums_out;
                t.m = (int)m; t.n = (int)n; t.k = (int)k; t.kq = (int)kq;
                t.n16 = (int)w->d.n16; t.ku = (int)w->d.ku; t.nb = (int)nb; t.nb_real = (int)w->d.nb_real;
                t.log2_block = w->d.log2_block; t.bits = w->bits; t.lut = w->lut ^ 0x80808080u; t.status = ds->status; t.ep = g.ep;
                e = lowbit_tc_launch(t, stream);
            } else if (mma) e = lowbit_mma_launch(g, w->bits, ds->sm_count, stream);
            else if ((int)m <= g_direct_rows && lowbit_direct_supported(g, false)) e = lowbit_direct_launch(g, w->bits, ds->sm_count, stream);
            else e = lowbit_gemv_launch(g, w->bits, ds->sm_count, stream);
        }
        if (e == cudaSuccess && q_out)
            e = cudaMemcpy2DAsync(q_out, k, aq.q, kq, k, m, cudaMemcpyDeviceToDevice, stream);
        if (e == cudaSuccess && sa_out)
            e = cudaMemcpy2DAsync(sa_out, w->d.nb_real * 4, aq.sa, nb * 4, w->d.nb_real * 4, m, cudaMemcpyDeviceToDevice, stream);
    }
    if (ext) cudaFreeAsync(ext, stream);
    if (ws) cudaFreeAsync(ws, stream);
    return e == cudaSuccess ? 0 : -6;
}

int smeg_matmul_lowbit_dev(const smeg_lowbit* w, const uint16_t* a, uint16_t* c, size_t m, const ep_desc16* ep, void* stream) {
    return lowbit_dev(w, a, c, m, ep, nullptr, nullptr, nullptr, (cudaStream_t)stream);
}
int smeg_matmul_lowbit_debug_dev(const smeg_lowbit* w, const uint16_t* a, uint16_t* c, size_t m, int8_t* q_out,
                                 float* sa_out, int32_t* sums_out, void* stream) {
    return lowbit_dev(w, a, c, m, nullptr, q_out, sa_out, sums_out, (cudaStream_t)stream);
}

// The 4-bit twin of a 2-bit / 1-bit weight set (see transcode.cu), built once under the
// handle's lock; the build synchronises, so it must not first happen inside a stream capture.
static int lowbit_twin(const smeg_lowbit* w, const smeg_q4** out) {
    smeg_q4* t = w->twin.load(std::memory_order_acquire);
    if (t) { *out = t; return 0; }
    if (w->bits == 2)
        for (int i = 0; i < 4; ++i)
            if (w->codebook[i] < -8 || w->codebook[i] > 7) return -3;
    std::lock_guard<std::mutex> lock(w->twin_lock);
    t = w->twin.load(std::memory_order_acquire);
    if (t) { *out = t; return 0; }
    if (!dev_state()) return -5;
    smeg_q4* h = new smeg_q4();
    h->d = make_dims(w->d.n, w->d.k, w->d.block, kQ4UnitDepth);
    h->code_bytes = h->d.n16 * h->d.ku * kUnitBytes;
    h->scale_elems = h->d.n16 * h->d.nb * 16;
    if ((h->code_bytes && cudaMalloc(&h->codes, h->code_bytes) != cudaSuccess) ||
        (h->scale_elems && cudaMalloc(&h->scales, h->scale_elems * 2) != cudaSuccess)) {
        smeg_q4_destroy(h);
        return -2;
    }
    LowbitToQ4Args a;
    a.src = w->codes; a.src_scales = w->scales; a.dst = h->codes; a.dst_scales = h->scales;
    a.n = w->d.n; a.k = w->d.k;
    a.ku_src = w->d.ku; a.n16_src = w->d.n16; a.nb_src = w->d.nb;
    a.ku4 = h->d.ku; a.nb4 = h->d.nb;
    a.dst_words = h->code_bytes / 4; a.dst_scale_elems = h->scale_elems;
    a.bits = w->bits; a.lut = w->lut;
    cudaStream_t s = nullptr;
    if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) { smeg_q4_destroy(h); return -2; }
    cudaError_t e = lowbit_to_q4_launch(a, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    cudaStreamDestroy(s);
    if (e != cudaSuccess) { smeg_q4_destroy(h); return -6; }
    w->twin.store(h, std::memory_order_release);
    *out = h;
    return 0;
}

static bool lowbit_needs_dense_twin(const smeg_lowbit* w) {
    if (w->bits != 2) return false;
    for (int i = 0; i < 4; ++i)
        if (w->codebook[i] < -8 || w->codebook[i] > 7) return true;
    return false;
}

// The dense f16 twin (see transcode.cu), built once under the handle's lock like the 4-bit one.
static int lowbit_twin_dense(const smeg_lowbit* w, const smeg_dense** out) {
    smeg_dense* t = w->twin_dense.load(std::memory_order_acquire);
    if (t) { *out = t; return 0; }
    std::lock_guard<std::mutex> lock(w->twin_lock);
    t = w->twin_dense.load(std::memory_order_acquire);
    if (t) { *out = t; return 0; }
    if (!dev_state()) return -5;
    smeg_dense* h = new smeg_dense();
    h->n = w->d.n; h->k = w->d.k; h->kd = (w->d.k + 7) / 8 * 8; h->bf16 = 0;
    const size_t elems = h->n * h->kd;
    if (cudaMalloc(&h->w, (elems ? elems : 8) * 2) != cudaSuccess) { smeg_dense_destroy(h); return -2; }
    LowbitToQ4Args a;
    memset(&a, 0, sizeof(a));
    a.src = w->codes; a.src_scales = w->scales; a.n = w->d.n; a.k = w->d.k;
    a.ku_src = w->d.ku; a.n16_src = w->d.n16; a.nb_src = w->d.nb; a.bits = w->bits; a.lut = w->lut;
    cudaStream_t s = nullptr;
    if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) { smeg_dense_destroy(h); return -2; }
    cudaError_t e = lowbit_to_dense_launch(a, h->w, h->kd, w->d.log2_block, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    cudaStreamDestroy(s);
    if (e != cudaSuccess) { smeg_dense_destroy(h); return -6; }
    w->twin_dense.store(h, std::memory_order_release);
    *out = h;
    return 0;
}

int smeg_lowbit_prepare_f16(const smeg_lowbit* w) {
    if (!w) return -4;
    if (lowbit_needs_dense_twin(w)) {
        const smeg_dense* d = nullptr;
        return lowbit_twin_dense(w, &d);
    }
    const smeg_q4* t = nullptr;
    return lowbit_twin(w, &t);
}

int smeg_matmul_lowbit_f16_dev(const smeg_lowbit* w, const uint16_t* a, uint16_t* c, size_t m, const ep_desc16* ep,
                               void* stream) {
    if (!w) return -4;
    if (m == 0 || w->d.n == 0) return 0;
    if (lowbit_needs_dense_twin(w)) {
        const smeg_dense* d = nullptr;
        const int rc = lowbit_twin_dense(w, &d);
        if (rc) return rc;
        return smeg_gemm_dense_dev(d, a, c, m, 0x3c00 /* beta = 1 */, 0, ep, stream);
    }
    const smeg_q4* t = nullptr;
    const int rc = lowbit_twin(w, &t);
    if (rc) return rc;
    return q4_dev(t, a, c, m, ep, 0, (cudaStream_t)stream);
}

// ---- dense 16-bit weights: prepack_f16 / prepack_bf16 + the Gemm builder's run ----
int smeg_dense_create(const uint16_t* b, size_t n, size_t k, int bf16, smeg_dense** out) {
    if (!out) return -4;
    *out = nullptr;
    if (mul_overflows(n, k) || ((n != 0 && k != 0) && !b)) return -4;
    if (!dev_state()) return -5;
    smeg_dense* h = new smeg_dense();
    h->n = n; h->k = k; h->kd = (k + 7) / 8 * 8; h->bf16 = bf16 ? 1 : 0;
    // b is k x n row-major (prepack_f16, src/kernels/f16.rs:212); the tensor cores take K-major rows
    std::vector<uint16_t> w(n * h->kd, 0);
    for (size_t d = 0; d < k; ++d)
        for (size_t j = 0; j < n; ++j) w[j * h->kd + d] = b[d * n + j];
    if (upload(w, &h->w)) { smeg_dense_destroy(h); return -2; }
    *out = h;
    return 0;
}
void smeg_dense_destroy(smeg_dense* w) {
    if (!w) return;
    if (w->w) cudaFree(w->w);
    delete w;
}
size_t smeg_dense_n(const smeg_dense* w) { return w->n; }
size_t smeg_dense_k(const smeg_dense* w) { return w->k; }

int smeg_gemm_dense_dev(const smeg_dense* w, const uint16_t* a, uint16_t* c, size_t m, uint16_t beta_bits, int col_major,
                        const ep_desc16* ep, void* stream_v) {
    if (!w) return -4;
    cudaStream_t stream = (cudaStream_t)stream_v;
    const size_t n = w->n, k = w->k;
    if (m == 0 || n == 0) return 0;
    if (!c || (k && !a) || m > 0x7fffffffu || n > 0x7fffffffu || k > 0x7fffffffu) return -4;
    DeviceState* ds = dev_state();
    if (!ds) return -5;
    if (k == 0) {
        // an empty depth: C = ep(T(0)) (the reference's k == 0 product is all zeros)
        return -3;
    }
    // the token tile travels by TMA: rows of 16-byte multiples at a 16-byte aligned base.  Any other A is
    // staged through a zero-padded copy [m][kd] (the weights are already padded to kd along K)
    uint16_t* a_pad = nullptr;
    if (k % 8 != 0 || ((uintptr_t)a & 15) != 0) {
        if (cudaMallocAsync(&a_pad, m * w->kd * 2, stream) != cudaSuccess) return -2;
        cudaError_t ce = cudaMemsetAsync(a_pad, 0, m * w->kd * 2, stream);
        if (ce == cudaSuccess) ce = cudaMemcpy2DAsync(a_pad, w->kd * 2, a, k * 2, k * 2, m, cudaMemcpyDeviceToDevice, stream);
        if (ce != cudaSuccess) { cudaFreeAsync(a_pad, stream); return -6; }
    }
    const uint16_t* a_run = a_pad ? a_pad : a;
    const size_t k_run = a_pad ? w->kd : k;
    if (!gemm_tc_supported(16, (int)m, (int)k_run, 5, a_run)) { if (a_pad) cudaFreeAsync(a_pad, stream); return -3; }
    GemmTcArgs t;
    memset(&t, 0, sizeof(t));
    EpNodeDev* ext = nullptr;
    int rc = make_ep(ep, n, &t.ep, stream, &ext);
    if (rc) { if (ext) cudaFreeAsync(ext, stream); if (a_pad) cudaFreeAsync(a_pad, stream); return rc; }
    t.wdense = w->w; t.kd = (int)w->kd; t.a = a_run; t.c = c;
    t.beta = w->bf16 ? __uint_as_float_host((uint32_t)beta_bits << 16) : h2f(beta_bits);
    t.col_major = col_major ? 1 : 0;
    t.m = (int)m; t.n = (int)n; t.k = (int)k_run;
    t.n16 = (int)((n + 15) / 16); t.ku = (int)((k_run + 63) / 64); t.nb = 0; t.log2_block = 5;
    t.status = ds->status;
    dim3 grid;
    size_t smem = 0, ws_floats = 0, ncounters = 0;
    gemm_tc_plan(t, ds->sm_count, &grid, &smem, &ws_floats, &ncounters);
    TcScratch sc;
    if (ws_floats && tc_scratch(stream, ws_floats, ncounters, &sc)) {
        if (ext) cudaFreeAsync(ext, stream);
        if (a_pad) cudaFreeAsync(a_pad, stream);
        return -2;
    }
    t.ws = sc.ws;
    t.counters = sc.counters;
    cudaError_t e = gemm_tc_launch(t, w->bf16, grid, smem, stream);
    if (ext) cudaFreeAsync(ext, stream);
    if (a_pad) cudaFreeAsync(a_pad, stream);
    return e == cudaSuccess ? 0 : -6;
}

int smeg_glu_f16_dev(uint16_t* out, const uint16_t* both, size_t m, size_t n, uint32_t act, void* stream) {
    if (act != SMEG_ACT_SILU && act != SMEG_ACT_GELU) return -4;
    return glu_launch(out, both, m, n, act, (cudaStream_t)stream) == cudaSuccess ? 0 : -6;
}
int smeg_add_f16_to_f32_dev(float* dst, const uint16_t* src, size_t len, void* stream) {
    return add_f16_to_f32_launch(dst, src, len, (cudaStream_t)stream) == cudaSuccess ? 0 : -6;
}
int smeg_act_f16_dev(uint16_t* dst, const uint16_t* src, size_t len, uint32_t act, void* stream) {
    return act_f16_launch(dst, src, len, act, (cudaStream_t)stream) == cudaSuccess ? 0 : -6;
}
int smeg_f32_to_f16_dev(uint16_t* dst, const float* src, size_t len, void* stream) {
    return f32_to_f16_launch(dst, src, len, (cudaStream_t)stream) == cudaSuccess ? 0 : -6;
}
int smeg_norm_rows_dev(uint16_t* y16, float* y32, const float* x, const float* weight, const float* bias, size_t rows, size_t dim,
                       float eps, int rms, void* stream) {
    if (rows == 0 || dim == 0) return 0;
    if ((!y16 && !y32) || !x || !weight || rows > 0x7fffffffu) return -4;
    if (!dev_state()) return -5;
    return norm_rows_launch(y16, y32, x, weight, bias, rows, dim, eps, rms ? 1 : 0, (cudaStream_t)stream) == cudaSuccess ? 0 : -6;
}
int smeg_rms_scales_dev(uint16_t* out, const uint16_t* x, size_t rows, size_t k, float eps, void* stream) {
    if (rows == 0) return 0;
    if (!out || !x || k == 0 || rows > 0x7fffffffu) return -4;
    if (!dev_state()) return -5;
    return rms_scales_launch(out, x, rows, k, eps, (cudaStream_t)stream) == cudaSuccess ? 0 : -6;
}
int smeg_f16_to_f32_dev(float* dst, const uint16_t* src, size_t len, void* stream) {
    return f16_to_f32_launch(dst, src, len, (cudaStream_t)stream) == cudaSuccess ? 0 : -6;
}

// ---------------------------------------------------------------------------
// host-pointer wrappers
// ---------------------------------------------------------------------------
}  // extern "C"
namespace {
// Device staging of a host-pointer call: stream-ordered allocations on the default stream, which the device's pool keeps
// cached between calls (its release threshold is raised when the device is first used), so that a call neither
// synchronises the device for an allocation nor returns memory to the driver.
struct DevBuf {
    void* p = nullptr;
    ~DevBuf() { if (p) cudaFreeAsync(p, 0); }
    int alloc(size_t bytes) { return cudaMallocAsync(&p, bytes ? bytes : 16, 0) == cudaSuccess ? 0 : -2; }
};

// status word check after a synchronous call
int finish_sync(DeviceState* ds) {
    if (cudaStreamSynchronize(0) != cudaSuccess) return -6;
    unsigned v = 0;
    if (cudaMemcpy(&v, ds->status, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return -6;
    if (v) {
        cudaMemset(ds->status, 0, sizeof(unsigned));
        reset_counters_after_timeout(ds->device);
        return -7;
    }
    return 0;
}

template <typename F>
int host_matmul(size_t m, size_t n, size_t k, const uint16_t* a, uint16_t* c, const ep_desc16* ep, F run) {
    if (m == 0 || n == 0) return 0;
    if (mul_overflows(m, k) || mul_overflows(m, n) || !c || (k && !a)) return -4;
    DeviceState* ds = dev_state();
    if (!ds) return -5;
    DevBuf da, dc;
    HostEp hep;
    if (da.alloc(m * k * 2) || dc.alloc(m * n * 2)) return -2;
    int rc = hep.build(ep, m, n);
    if (rc) return rc;
    if (k && cudaMemcpy(da.p, a, m * k * 2, cudaMemcpyHostToDevice) != cudaSuccess) return -6;
    rc = run((const uint16_t*)da.p, (uint16_t*)dc.p, hep.get());
    if (rc) return rc;
    rc = finish_sync(ds);
    if (rc) return rc;
    if (cudaMemcpy(c, dc.p, m * n * 2, cudaMemcpyDeviceToHost) != cudaSuccess) return -6;
    return 0;
}
}  // namespace
extern "C" {

int smeg_matmul_q4_f16(const smeg_q4* w, const uint16_t* a, uint16_t* c, size_t m, const ep_desc16* ep) {
    if (!w) return -4;
    TraceScope ts("matmul_q4_f16", m, w->d.n, w->d.k);
    return host_matmul(m, w->d.n, w->d.k, a, c, ep, [&](const uint16_t* da, uint16_t* dc, const ep_desc16* dep) {
        return q4_dev(w, da, dc, m, dep, 0, 0);
    });
}
int smeg_matmul_q4_bf16(const smeg_q4* w, const uint16_t* a, uint16_t* c, size_t m, const ep_desc16* ep) {
    if (!w) return -4;
    TraceScope ts("matmul_q4_bf16", m, w->d.n, w->d.k);
    return host_matmul(m, w->d.n, w->d.k, a, c, ep, [&](const uint16_t* da, uint16_t* dc, const ep_desc16* dep) {
        return q4_dev(w, da, dc, m, dep, 1, 0);
    });
}
int smeg_matmul_lowbit(const smeg_lowbit* w, const uint16_t* a, uint16_t* c, size_t m, const ep_desc16* ep) {
    if (!w) return -4;
    TraceScope ts(w->bits == 2 ? "matmul_q2" : "matmul_q1", m, w->d.n, w->d.k);
    return host_matmul(m, w->d.n, w->d.k, a, c, ep, [&](const uint16_t* da, uint16_t* dc, const ep_desc16* dep) {
        return lowbit_dev(w, da, dc, m, dep, nullptr, nullptr, nullptr, 0);
    });
}
int smeg_matmul_lowbit_f16(const smeg_lowbit* w, const uint16_t* a, uint16_t* c, size_t m, const ep_desc16* ep) {
    if (!w) return -4;
    TraceScope ts(w->bits == 2 ? "matmul_q2_mopa" : "matmul_q1_mopa", m, w->d.n, w->d.k);
    return host_matmul(m, w->d.n, w->d.k, a, c, ep, [&](const uint16_t* da, uint16_t* dc, const ep_desc16* dep) {
        return smeg_matmul_lowbit_f16_dev(w, da, dc, m, dep, nullptr);
    });
}
int smeg_gemm_dense(const smeg_dense* w, const uint16_t* a, uint16_t* c, size_t m, uint16_t beta_bits, int col_major,
                    const ep_desc16* ep) {
    if (!w) return -4;
    TraceScope ts(w->bf16 ? "gemm_bf16_packed" : "gemm_f16_packed", m, w->n, w->k);
    return host_matmul(m, w->n, w->k, a, c, ep, [&](const uint16_t* da, uint16_t* dc, const ep_desc16* dep) {
        return smeg_gemm_dense_dev(w, da, dc, m, beta_bits, col_major, dep, nullptr);
    });
}

// ---------------------------------------------------------------------------
// MLP block
// ---------------------------------------------------------------------------
// ---- attention against an f16 KV cache ----
int smeg_kv_append_dev(uint16_t* k_cache, uint16_t* v_cache, const uint16_t* src, size_t src_stride, size_t k_off, size_t v_off,
                       size_t row_len, size_t pos, size_t rows, void* stream) {
    if (rows == 0 || row_len == 0) return 0;
    if (!k_cache || !v_cache || !src || k_off + row_len > src_stride || v_off + row_len > src_stride) return -4;
    if (!dev_state()) return -5;
    return kv_append_launch(k_cache, v_cache, src, src_stride, k_off, v_off, row_len, pos, rows, (cudaStream_t)stream) == cudaSuccess ? 0 : -6;
}
int smeg_attn_kv_causal_dev(float* out, const void* q, int q_f32, size_t q_stride, const uint16_t* k, const uint16_t* v, size_t start,
                            size_t rows, size_t heads, size_t kv_heads, size_t head_dim, float scale, void* stream) {
    if (rows == 0) return 0;
    // the reference's panics (src/kernels/kv_attention.rs:171-199) as rc -4
    if (!out || !q || !k || !v) return -4;
    if (head_dim % 8 != 0 || head_dim < 8 || head_dim > 256) return -4;
    if (kv_heads == 0 || heads == 0 || heads % kv_heads != 0 || q_stride < heads * head_dim) return -4;
    if (((uintptr_t)k & 15) != 0 || ((uintptr_t)v & 15) != 0) return -4;
    if (start + rows > 0x7fffffffu || heads > 65535 || rows > 65535) return -3;
    if (!dev_state()) return -5;
    AttnArgs a;
    memset(&a, 0, sizeof(a));
    a.out = out; a.q = q; a.q_stride = q_stride; a.k = k; a.v = v;
    a.start = (int)start; a.rows = (int)rows; a.heads = (int)heads; a.kv_heads = (int)kv_heads; a.head_dim = (int)head_dim;
    a.scale = scale;
    const cudaError_t e = attn_kv_causal_launch(a, q_f32, (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : (e == cudaErrorInvalidValue ? -3 : -6);
}

int smeg_mlp_create(const smeg_q4* gate_up, const smeg_q4* down, uint32_t gate_act, smeg_mlp** out) {
    if (!out || !gate_up || !down) return -4;
    *out = nullptr;
    if (gate_act != SMEG_ACT_SILU && gate_act != SMEG_ACT_GELU) return -4;
    if (gate_up->d.n % 2 != 0 || down->d.k != gate_up->d.n / 2) return -4;   // "down takes up's outputs"
    if (gate_up->affine || down->affine) return -3;                          // the block's fused forms take Q4_0 weights
    smeg_mlp* h = new smeg_mlp{gate_up, down, gate_act};
    *out = h;
    return 0;
}
void smeg_mlp_destroy(smeg_mlp* mlp) { delete mlp; }

// both = x @ gate_up (f16), hid = glu(both), then the down projection either
// rounded to f16 and added into y (partial == nullptr) or left as f32 partial sums.
static int mlp_run(smeg_mlp* mlp, const uint16_t* x, float* y, float* partial, size_t m, cudaStream_t stream, const TpPush* push = nullptr) {
    if (!mlp) return -4;
    if (m == 0) return 0;
    const size_t h = mlp->down->d.k, d_out = mlp->down->d.n;
    if (mul_overflows(m, 2 * h)) return -4;
    char* ws = nullptr;
    const size_t both_bytes = (m * 2 * h * 2 + 255) / 256 * 256, hid_bytes = (m * h * 2 + 255) / 256 * 256;
    const size_t out_bytes = (m * d_out * 2 + 255) / 256 * 256;
    // prefill-sized batches: the gated product is formed in the gate/up GEMM's drain and the residual add in the
    // down GEMM's, with the arithmetic of the separate passes (two launches instead of four)
    if (push && !(m > 64)) return -3;
    const bool fuse = m > 64 && h % 32 == 0 && mlp->gate_up->d.n == 2 * h && q4_uses_tc(mlp->gate_up, x, m) &&
                      mlp->down->d.k % 8 == 0 && (int)m > g_tc_min_rows && mlp->down->d.log2_block >= 3;
    if (cudaMallocAsync(&ws, (fuse ? 0 : both_bytes) + hid_bytes + out_bytes, stream) != cudaSuccess) return -2;
    uint16_t* hid = (uint16_t*)ws;
    uint16_t* out = (uint16_t*)(ws + hid_bytes);
    uint16_t* both = (uint16_t*)(ws + hid_bytes + out_bytes);
    int rc;
    if (fuse) {
        rc = q4_dev(mlp->gate_up, x, hid, m, nullptr, 0, stream, nullptr, (int)mlp->act);
        if (!rc) rc = partial ? q4_dev(mlp->down, hid, nullptr, m, nullptr, 0, stream, partial, 0, nullptr, push)
                              : q4_dev(mlp->down, hid, nullptr, m, nullptr, 0, stream, nullptr, 0, y);
    } else if (q4_takes_direct(mlp->gate_up, x, m, 0, (int)mlp->act) && q4_takes_direct(mlp->down, hid, m, 0, 0) && mlp->gate_up->d.n == 2 * h) {
        // decode-sized steps on the one-wave kernels: the gated product is formed where the gate/up projection's sums
        // meet and the residual add where the down projection's do (two launches instead of four, the same arithmetic)
        rc = q4_dev(mlp->gate_up, x, hid, m, nullptr, 0, stream, nullptr, (int)mlp->act);
        if (!rc) rc = partial ? q4_dev(mlp->down, hid, nullptr, m, nullptr, 0, stream, partial)
                              : q4_dev(mlp->down, hid, nullptr, m, nullptr, 0, stream, nullptr, 0, y);
    } else {
        rc = q4_dev(mlp->gate_up, x, both, m, nullptr, 0, stream);
        if (!rc) rc = glu_launch(hid, both, m, h, mlp->act, stream) == cudaSuccess ? 0 : -6;
        if (!rc) {
            if (partial) {
                rc = push ? -3 : q4_dev(mlp->down, hid, nullptr, m, nullptr, 0, stream, partial);
            } else {
                rc = q4_dev(mlp->down, hid, out, m, nullptr, 0, stream);
                if (!rc) rc = add_f16_to_f32_launch(y, out, m * d_out, stream) == cudaSuccess ? 0 : -6;
            }
        }
    }
    cudaFreeAsync(ws, stream);
    return rc;
}

int smeg_mlp_accumulate_dev(smeg_mlp* mlp, const uint16_t* x, float* y, size_t m, void* stream) {
    return mlp_run(mlp, x, y, nullptr, m, (cudaStream_t)stream);
}
int smeg_mlp_partial_dev(smeg_mlp* mlp, const uint16_t* x, float* partial, size_t m, void* stream) {
    return mlp_run(mlp, x, nullptr, partial, m, (cudaStream_t)stream);
}
int smeg_mlp_partial_push_dev(smeg_mlp* mlp, const uint16_t* x, const uint64_t* buf_ptrs, int rank, int world, size_t m, void* stream) {
    if (!mlp || !buf_ptrs || world < 2 || world > 8 || rank < 0 || rank >= world) return -4;
    TpPush push;
    memset(&push, 0, sizeof(push));
    for (int s = 0; s < world; ++s) {
        if (!buf_ptrs[s] || (buf_ptrs[s] & 15) != 0) return -4;
        push.bufs[s] = reinterpret_cast<float*>(buf_ptrs[s]);
    }
    push.world = world; push.rank = rank; push.rows = (int)((m + world - 1) / world);
    return mlp_run(mlp, x, nullptr, push.bufs[rank], m, (cudaStream_t)stream, &push);
}
int smeg_mlp_finish_dev(float* y, const float* sum, size_t len, void* stream) {
    return round_add_f32_launch(y, sum, len, (cudaStream_t)stream) == cudaSuccess ? 0 : -6;
}
int smeg_mlp_reduce_finish_dev(float* y, const uint64_t* buf_ptrs, const uint64_t* flag_ptrs, int rank, int world,
                               size_t len, uint32_t seq, int oneshot, void* stream) {
    if (len == 0) return 0;
    if (!y || !buf_ptrs || !flag_ptrs || world < 1 || rank < 0 || rank >= world) return -4;
    if (world > 8 || len % 4 != 0 || ((uintptr_t)y & 15) != 0) return -3;
    DeviceState* ds = dev_state();
    if (!ds) return -5;
    TpReduceArgs a;
    memset(&a, 0, sizeof(a));
    for (int s = 0; s < world; ++s) {
        if (!buf_ptrs[s] || !flag_ptrs[s] || (buf_ptrs[s] & 15) != 0 || (flag_ptrs[s] & 3) != 0) return -4;
        a.bufs[s] = reinterpret_cast<float*>(buf_ptrs[s]);
        a.flags[s] = reinterpret_cast<uint32_t*>(flag_ptrs[s]);
    }
    a.y = y; a.rank = rank; a.world = world; a.len = len; a.seq = seq; a.status = ds->status;
    a.oneshot = oneshot ? 1 : 0;
    a.res_off = len;
    return tp_reduce_finish_launch(a, ds->sm_count, (cudaStream_t)stream) == cudaSuccess ? 0 : -6;
}
int smeg_mlp_reduce_finish_pushed_dev(float* y, const uint64_t* buf_ptrs, const uint64_t* flag_ptrs, int rank, int world,
                                      size_t m, size_t d, uint32_t seq, void* stream) {
    if (m == 0 || d == 0) return 0;
    if (!y || !buf_ptrs || !flag_ptrs || world < 2 || rank < 0 || rank >= world) return -4;
    if (world > 8 || d % 4 != 0 || ((uintptr_t)y & 15) != 0) return -3;
    DeviceState* ds = dev_state();
    if (!ds) return -5;
    TpReduceArgs a;
    memset(&a, 0, sizeof(a));
    for (int s = 0; s < world; ++s) {
        if (!buf_ptrs[s] || !flag_ptrs[s] || (buf_ptrs[s] & 15) != 0 || (flag_ptrs[s] & 3) != 0) return -4;
        a.bufs[s] = reinterpret_cast<float*>(buf_ptrs[s]);
        a.flags[s] = reinterpret_cast<uint32_t*>(flag_ptrs[s]);
    }
    const size_t rows = (m + world - 1) / world;
    a.y = y; a.rank = rank; a.world = world; a.len = m * d; a.seq = seq; a.status = ds->status;
    a.pushed = 1; a.slice = rows * d; a.res_off = (size_t)world * rows * d;
    return tp_reduce_finish_launch(a, ds->sm_count, (cudaStream_t)stream) == cudaSuccess ? 0 : -6;
}
int smeg_mlp_accumulate(smeg_mlp* mlp, const uint16_t* x, float* y, size_t m) {
    if (!mlp) return -4;
    if (m == 0) return 0;
    DeviceState* ds = dev_state();
    if (!ds) return -5;
    const size_t k = mlp->gate_up->d.k, d_out = mlp->down->d.n;
    TraceScope ts("mlp_accumulate", m, d_out, k);
    DevBuf dx, dy;
    if (dx.alloc(m * k * 2) || dy.alloc(m * d_out * 4)) return -2;
    if (cudaMemcpy(dx.p, x, m * k * 2, cudaMemcpyHostToDevice) != cudaSuccess) return -6;
    if (cudaMemcpy(dy.p, y, m * d_out * 4, cudaMemcpyHostToDevice) != cudaSuccess) return -6;
    int rc = mlp_run(mlp, (const uint16_t*)dx.p, (float*)dy.p, nullptr, m, 0);
    if (rc) return rc;
    rc = finish_sync(ds);
    if (rc) return rc;
    if (cudaMemcpy(y, dy.p, m * d_out * 4, cudaMemcpyDeviceToHost) != cudaSuccess) return -6;
    return 0;
}

// ---------------------------------------------------------------------------
// drop-in entry points (the reference's signatures, band-major host arrays)
// ---------------------------------------------------------------------------
}  // extern "C"
namespace {
struct CacheKey {
    const void* ptr; size_t n, k, block; int kind;
    bool operator<(const CacheKey& o) const {
        return std::tie(ptr, n, k, block, kind) < std::tie(o.ptr, o.n, o.k, o.block, o.kind);
    }
};
struct CacheVal { smeg_q4* q4 = nullptr; smeg_lowbit* lb = nullptr; };
std::mutex g_cache_mu;
std::map<CacheKey, CacheVal> g_cache;
}  // namespace
extern "C" {

static smeg_q4* cached_q4(const uint8_t* nibbles, const uint16_t* scales, const uint16_t* mins, size_t n, size_t k,
                          size_t block, int* rc) {
    std::lock_guard<std::mutex> lk(g_cache_mu);
    CacheKey key{nibbles, n, k, block, 4};
    auto it = g_cache.find(key);
    if (it != g_cache.end()) { *rc = 0; return it->second.q4; }
    smeg_q4* h = nullptr;
    *rc = smeg_q4_from_band(nibbles, scales, mins, n, k, block, &h);
    if (*rc) return nullptr;
    g_cache[key].q4 = h;
    return h;
}
static smeg_lowbit* cached_lowbit(int bits, const uint8_t* packed, const uint16_t* scales, const int8_t* codebook,
                                  size_t n, size_t k, size_t block, int* rc) {
    std::lock_guard<std::mutex> lk(g_cache_mu);
    CacheKey key{packed, n, k, block, bits};
    auto it = g_cache.find(key);
    if (it != g_cache.end() && (bits == 1 || memcmp(it->second.lb->codebook, codebook, 4) == 0)) { *rc = 0; return it->second.lb; }
    if (it != g_cache.end()) { smeg_lowbit_destroy(it->second.lb); g_cache.erase(it); }
    smeg_lowbit* h = nullptr;
    *rc = bits == 2 ? smeg_q2_from_band(packed, scales, n, k, block, codebook, &h)
                    : smeg_q1_from_band(packed, scales, n, k, block, &h);
    if (*rc) return nullptr;
    g_cache[key].lb = h;
    return h;
}

void smeg_forget(const void* packed) {
    std::lock_guard<std::mutex> lk(g_cache_mu);
    for (auto it = g_cache.begin(); it != g_cache.end();) {
        if (it->first.ptr == packed) {
            if (it->second.q4) smeg_q4_destroy(it->second.q4);
            if (it->second.lb) smeg_lowbit_destroy(it->second.lb);
            it = g_cache.erase(it);
        } else ++it;
    }
}

int gemm_sme_f16f16_q4(size_t m, size_t n, size_t k, uint16_t* dst, const uint16_t* lhs, const uint8_t* nibbles,
                       const uint16_t* scales, const uint16_t* mins, size_t block, const ep_desc16* ep) {
    if (m == 0 || n == 0) return 0;
    int rc = 0;
    smeg_q4* w = cached_q4(nibbles, scales, mins, n, k, block, &rc);
    if (!w) return rc;
    return smeg_matmul_q4_f16(w, lhs, dst, m, ep);
}
int gemm_sme_b16b16_q4(size_t m, size_t n, size_t k, uint16_t* dst, const uint16_t* lhs, const uint8_t* nibbles,
                       const uint16_t* scales, const uint16_t* mins, const uint16_t* scales_bf16,
                       const uint16_t* mins_bf16, size_t block, const ep_desc16* ep) {
    (void)scales_bf16; (void)mins_bf16;
    if (m == 0 || n == 0) return 0;
    int rc = 0;
    smeg_q4* w = cached_q4(nibbles, scales, mins, n, k, block, &rc);
    if (!w) return rc;
    return smeg_matmul_q4_bf16(w, lhs, dst, m, ep);
}
int gemm_sme_f16_q1(size_t m, size_t n, size_t k, uint16_t* dst, const uint16_t* lhs, const uint8_t* signs,
                    const uint16_t* scales, size_t block, const ep_desc16* ep) {
    if (m == 0 || n == 0) return 0;
    int rc = 0;
    smeg_lowbit* w = cached_lowbit(1, signs, scales, nullptr, n, k, block, &rc);
    if (!w) return rc;
    return smeg_matmul_lowbit(w, lhs, dst, m, ep);
}
int gemm_sme_f16_q2(size_t m, size_t n, size_t k, uint16_t* dst, const uint16_t* lhs, const uint8_t* codes,
                    const uint16_t* scales, const int8_t* codebook, size_t block, const ep_desc16* ep) {
    if (m == 0 || n == 0) return 0;
    if (!codebook) return -4;
    int rc = 0;
    smeg_lowbit* w = cached_lowbit(2, codes, scales, codebook, n, k, block, &rc);
    if (!w) return rc;
    return smeg_matmul_lowbit(w, lhs, dst, m, ep);
}

int gemm_sme_f16f16_q1(size_t m, size_t n, size_t k, uint16_t* dst, const uint16_t* lhs, const uint8_t* signs,
                       const uint16_t* scales, size_t block, const ep_desc16* ep) {
    if (m == 0 || n == 0) return 0;
    int rc = 0;
    smeg_lowbit* w = cached_lowbit(1, signs, scales, nullptr, n, k, block, &rc);
    if (!w) return rc;
    return smeg_matmul_lowbit_f16(w, lhs, dst, m, ep);
}
int gemm_sme_f16f16_q2(size_t m, size_t n, size_t k, uint16_t* dst, const uint16_t* lhs, const uint8_t* codes,
                       const uint16_t* scales, const int8_t* codebook, size_t block, const ep_desc16* ep) {
    if (m == 0 || n == 0) return 0;
    if (!codebook) return -4;
    int rc = 0;
    smeg_lowbit* w = cached_lowbit(2, codes, scales, codebook, n, k, block, &rc);
    if (!w) return rc;
    return smeg_matmul_lowbit_f16(w, lhs, dst, m, ep);
}

void neon_glu_f16(uint16_t* out, const uint16_t* in, size_t m, size_t n, uint32_t act) {
    if (m * n == 0 || !dev_state()) return;
    DevBuf di, dout;
    if (di.alloc(m * 2 * n * 2) || dout.alloc(m * n * 2)) return;
    if (cudaMemcpy(di.p, in, m * 2 * n * 2, cudaMemcpyHostToDevice) != cudaSuccess) return;
    if (glu_launch((uint16_t*)dout.p, (const uint16_t*)di.p, m, n, act, 0) != cudaSuccess) return;
    cudaMemcpy(out, dout.p, m * n * 2, cudaMemcpyDeviceToHost);
}
void neon_act_f16(uint16_t* dst, const uint16_t* src, size_t n, uint32_t act) {
    if (n == 0 || !dev_state()) return;
    DevBuf dd, dsrc;
    if (dd.alloc(n * 2) || dsrc.alloc(n * 2)) return;
    if (cudaMemcpy(dsrc.p, src, n * 2, cudaMemcpyHostToDevice) != cudaSuccess) return;
    if (act_f16_launch((uint16_t*)dd.p, (const uint16_t*)dsrc.p, n, act, 0) != cudaSuccess) return;
    cudaMemcpy(dst, dd.p, n * 2, cudaMemcpyDeviceToHost);
}
void neon_f32_to_f16(uint16_t* dst, const float* src, size_t n) {
    if (n == 0 || !dev_state()) return;
    DevBuf dd, dsrc;
    if (dd.alloc(n * 2) || dsrc.alloc(n * 4)) return;
    if (cudaMemcpy(dsrc.p, src, n * 4, cudaMemcpyHostToDevice) != cudaSuccess) return;
    if (f32_to_f16_launch((uint16_t*)dd.p, (const float*)dsrc.p, n, 0) != cudaSuccess) return;
    cudaMemcpy(dst, dd.p, n * 2, cudaMemcpyDeviceToHost);
}
void neon_f16_to_f32(float* dst, const uint16_t* src, size_t n) {
    if (n == 0 || !dev_state()) return;
    DevBuf dd, dsrc;
    if (dd.alloc(n * 4) || dsrc.alloc(n * 2)) return;
    if (cudaMemcpy(dsrc.p, src, n * 2, cudaMemcpyHostToDevice) != cudaSuccess) return;
    if (f16_to_f32_launch((float*)dd.p, (const uint16_t*)dsrc.p, n, 0) != cudaSuccess) return;
    cudaMemcpy(dst, dd.p, n * 4, cudaMemcpyDeviceToHost);
}
void neon_add_f16_to_f32(float* dst, const uint16_t* src, size_t n) {
    if (n == 0 || !dev_state()) return;
    DevBuf dd, dsrc;
    if (dd.alloc(n * 4) || dsrc.alloc(n * 2)) return;
    if (cudaMemcpy(dd.p, dst, n * 4, cudaMemcpyHostToDevice) != cudaSuccess) return;
    if (cudaMemcpy(dsrc.p, src, n * 2, cudaMemcpyHostToDevice) != cudaSuccess) return;
    if (add_f16_to_f32_launch((float*)dd.p, (const uint16_t*)dsrc.p, n, 0) != cudaSuccess) return;
    cudaMemcpy(dst, dd.p, n * 4, cudaMemcpyDeviceToHost);
}

}  // extern "C"
