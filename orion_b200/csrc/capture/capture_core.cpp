// Client side of the capture protocol: thread -> client mapping, the gate every
// interposed call passes through, and the two control calls client scripts make
// (`block`, `stop`).
//
// Reference behaviour being replaced: get_idx / block in
// src/cuda_capture/utils_interc.cpp:3-64 and the exported block(int)/stop() in
// src/cuda_capture/intercept_temp.cpp:124-142.
#include "capture_core.h"

#include <dlfcn.h>
#include <sched.h>
#include <stdio.h>
#include <stdlib.h>
#include <sys/syscall.h>
#include <time.h>
#include <unistd.h>

#if defined(__x86_64__)
#include <immintrin.h>
#define ORION_PAUSE() _mm_pause()
#else
#define ORION_PAUSE() ((void)0)
#endif

static orion_shared g_shared;

extern "C" orion_shared* orion_capture_shared(void) {
    g_shared.abi_version = ORION_CAPTURE_ABI_VERSION;
    return &g_shared;
}

// ORION_CAPTURE_STATS=1: print the per-type call counts when the process exits.
__attribute__((constructor)) static void orion_capture_ctor() {
    const char* e = getenv("ORION_CAPTURE_STATS");
    if (e && atoi(e)) {
        atexit([] {
            fprintf(stderr, "orion capture: seen/scheduled per record type:");
            for (int t = 0; t < ORION_REC_TYPE_COUNT; t++)
                if (g_shared.seen[t].load()) fprintf(stderr, " %d:%llu/%llu", t, (unsigned long long)g_shared.seen[t].load(),
                                                     (unsigned long long)g_shared.captured[t].load());
            fprintf(stderr, " passthrough:%llu\n", (unsigned long long)g_shared.passthrough.load());
        });
    }
}

namespace orion_capture {

static thread_local int tls_idx = -1;
static thread_local int tls_epoch = -1;
static thread_local int tls_tid = 0;
static thread_local int tls_last_quota = 0;      // SM quota of the calling thread's latest grant
static thread_local bool tls_in_gate = false;   // a call made while this thread is already inside a gate passes through

static inline int my_tid() {
    if (!tls_tid) tls_tid = (int)syscall(SYS_gettid);
    return tls_tid;
}

// Pin a client thread the first time it is seen, like the reference
// (utils_interc.cpp:36-49), but only when the scheduler asked for it and with an
// offset it chose (several replicas on one host must not share cores).
static void maybe_pin(int slot, int idx) {
    orion_shared& sh = g_shared;
    if (!sh.pin_threads || sh.affinity_set[slot].load(std::memory_order_relaxed)) return;
    cpu_set_t mask;
    CPU_ZERO(&mask);
    if (sh.n_cores > 0) CPU_SET(sh.core_list[(1 + idx) % sh.n_cores], &mask);
    else CPU_SET(sh.core_offset + idx, &mask);
    if (sched_setaffinity(0, sizeof(mask), &mask) != 0) perror("orion: sched_setaffinity");
    sh.affinity_set[slot].store(1, std::memory_order_relaxed);
}

int client_index_of_thread() {
    orion_shared& sh = g_shared;
    if (!sh.active.load(std::memory_order_acquire)) return -1;
    int ep = sh.epoch.load(std::memory_order_acquire);
    if (ep == tls_epoch) return tls_idx;
    int tid = my_tid();
    int idx = -1;
    for (int i = 0; i < ORION_MAX_THREADS; i++) {
        if (sh.thread_ids[i].load(std::memory_order_relaxed) == tid) {
            idx = sh.thread_client[i].load(std::memory_order_relaxed);
            if (idx >= 0 && idx < sh.num_clients) maybe_pin(i, idx);
            break;
        }
    }
    if (idx >= sh.num_clients) idx = -1;   // the scheduler's own thread passes through
    tls_idx = idx;
    tls_epoch = ep;
    return idx;
}

int client_index_of_stream(void* stream) {
    orion_shared& sh = g_shared;
    if (!stream || !sh.active.load(std::memory_order_acquire)) return -1;
    for (int i = 0; i < sh.num_clients; i++)
        if (sh.client_stream[i] == stream) return i;
    return -1;
}

// Elastic kernels: a small open-addressing table of device-function pointers, written rarely
// (once per kernel, the first time its library launches it) and read on every granted launch.
static constexpr int kElasticSlots = 256;
static std::atomic<uintptr_t> g_elastic_func[kElasticSlots];
static std::atomic<int> g_elastic_factor[kElasticSlots];

static inline unsigned elastic_hash(uintptr_t f) { return (unsigned)((f >> 4) * 2654435761u) % kElasticSlots; }

static int elastic_factor_of(const void* func) {
    const uintptr_t f = (uintptr_t)func;
    unsigned h = elastic_hash(f);
    for (int probe = 0; probe < kElasticSlots; probe++, h = (h + 1) % kElasticSlots) {
        uintptr_t cur = g_elastic_func[h].load(std::memory_order_acquire);
        if (cur == f) return g_elastic_factor[h].load(std::memory_order_acquire);
        if (cur == 0) return 0;
    }
    return 0;
}

unsigned clamp_grid(const void* func, unsigned grid_x, int num_ctas) {
    if (num_ctas <= 0) return grid_x;
    const int factor = elastic_factor_of(func);
    if (factor <= 0) return grid_x;
    const unsigned long long cap = (unsigned long long)num_ctas * (unsigned)factor;
    if (grid_x <= cap) return grid_x;
    g_shared.clamped_launches.fetch_add(1, std::memory_order_relaxed);
    return (unsigned)cap;
}

static inline int64_t mono_ms() {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (int64_t)ts.tv_sec * 1000 + ts.tv_nsec / 1000000;
}
static inline int64_t gate_timeout_ms() {
    static int64_t v = [] {
        const char* e = getenv("ORION_GATE_TIMEOUT_S");
        return (int64_t)(e ? atoi(e) : 30) * 1000;
    }();
    return v;
}

static inline bool is_default_stream(void* s) {
    uintptr_t v = (uintptr_t)s;
    return v == 0 || v == 1 || v == 2;   // NULL, cudaStreamLegacy, cudaStreamPerThread
}

// A client's ring has one producer at a time.  Several threads can act for one client (its registered thread, the autograd
// thread replaying its stream, registered helpers); they take turns here, from the push of a record to the launch behind its
// grant, so that records, grants and events stay paired.  Uncontended in the clients of the benchmark (forward and backward
// of one client never overlap).
static std::atomic<uint32_t> g_producer_lock[ORION_MAX_CLIENTS];
// Set when a client gave up waiting for a grant while nobody was polling (a pause between two phases of the scheduler that
// the client's op stream did not expect, e.g. a profile with fewer rows than the client launches ops): its further ops of the
// same pause run unscheduled at once instead of waiting out the timeout one by one.  Cleared when polling is seen again and
// at the end of the client's request (block).
static std::atomic<uint32_t> g_gave_up_in_pause[ORION_MAX_CLIENTS];

bool gate_begin(Gate* g, int type, void* user_stream, uint64_t tag) {
    orion_shared& sh = g_shared;
    if (tls_in_gate) return false;
    sh.seen[type & 31].fetch_add(1, std::memory_order_relaxed);
    g->launch = nullptr;
    int idx = client_index_of_thread();
    if (idx < 0) idx = client_index_of_stream(user_stream);   // e.g. the autograd thread replaying a client's stream
    if (idx < 0) {
        if (sh.active.load(std::memory_order_relaxed)) sh.passthrough.fetch_add(1, std::memory_order_relaxed);
        if (profile_enabled()) {   // unscheduled profiling run: time the call on the caller's stream
            g->idx = -2;
            g->seq = 0;
            g->stream = user_stream;
            g->event = nullptr;
            g->num_ctas = 0;
            g->type = type;
            g->tag = tag;
            tls_in_gate = true;
            profile_begin(g);
            return true;
        }
        return false;
    }
    orion_ring& r = sh.rings[idx];
    for (uint32_t spins = 0; g_producer_lock[idx].exchange(1, std::memory_order_acquire) != 0;) {
        ORION_PAUSE();
        if ((++spins & 0x3f) == 0) sched_yield();
    }
    uint64_t seq = r.tail.load(std::memory_order_relaxed);
    orion_record& rec = r.recs[seq % ORION_RING_CAP];
    rec.type = type;
    rec.flags = 0;
    rec.tag = tag;
    r.tail.store(seq + 1, std::memory_order_release);
    sh.captured[type & 31].fetch_add(1, std::memory_order_relaxed);

    // Wait for the grant.  The high-priority client (last index) spins; best-effort
    // clients yield the core now and then so that they do not starve it.
    const bool hp = idx == sh.num_clients - 1;
    const bool memop = orion_is_memop(type) != 0;
    uint32_t spins = 0;
    int64_t t0 = 0;
    bool self_granted = false;
    while (r.granted.load(std::memory_order_acquire) <= seq) {
        bool take = false;
        const bool polling = sh.polling.load(std::memory_order_acquire) != 0;
        if (polling && g_gave_up_in_pause[idx].load(std::memory_order_relaxed))   // read-only in the common case: no line bouncing
            g_gave_up_in_pause[idx].store(0, std::memory_order_relaxed);
        if (!sh.active.load(std::memory_order_acquire)) {
            take = true;   // scheduler detached while we were queued: run the call unscheduled
        } else if (memop && !polling) {
            take = true;   // nobody polls between two phases; memory operations need no decision
        } else if (!polling && g_gave_up_in_pause[idx].load(std::memory_order_relaxed)) {
            take = true;   // this pause already cost the client one full timeout
        } else if ((++spins & 0xfffff) == 0) {
            int64_t now = mono_ms();
            if (!t0) t0 = now;
            if (now - t0 > gate_timeout_ms()) {
                fprintf(stderr, "orion: client %d waited more than %lld ms for a grant (record type %d, seq %llu, polling %d); "
                                "running the call unscheduled\n", idx, (long long)gate_timeout_ms(), type,
                        (unsigned long long)seq, sh.polling.load());
                sh.wait_timeouts.fetch_add(1);
                if (!sh.polling.load(std::memory_order_acquire)) g_gave_up_in_pause[idx].store(1, std::memory_order_relaxed);
                take = true;
            }
        }
        if (take) {
            uint64_t expect = seq;
            if (r.granted.compare_exchange_strong(expect, seq + 1, std::memory_order_acq_rel)) self_granted = true;
            break;   // if the exchange failed the scheduler granted meanwhile
        }
        ORION_PAUSE();
        if (!hp && (spins & 0x3ff) == 0) sched_yield();
    }
    tls_in_gate = true;
    g->idx = idx;
    g->seq = seq;
    g->type = type;
    g->tag = tag;
    g->event = self_granted ? nullptr : r.grant.event;
    g->num_ctas = self_granted ? 0 : r.grant.num_ctas;
    tls_last_quota = g->num_ctas;
    void* granted_stream = self_granted ? sh.client_stream[idx] : r.grant.stream;
    g->stream = is_default_stream(user_stream) ? granted_stream : user_stream;
    return true;
}

void gate_end(Gate* g) {
    tls_in_gate = false;
    if (g->idx == -2) {
        profile_end(g);
        return;
    }
    orion_ring& r = g_shared.rings[g->idx];
    if (g->event) real_event_record(g->event, g->stream);
    r.submitted.store(g->seq + 1, std::memory_order_release);
    g_producer_lock[g->idx].store(0, std::memory_order_release);
}

}  // namespace orion_capture

using namespace orion_capture;

extern "C" {

// Client waits until request `it` has completed on the GPU (intercept_temp.cpp:125-130).
void block(int it) {
    orion_shared& sh = g_shared;
    profile_mark_iteration(it);
    int idx = client_index_of_thread();
    if (idx < 0) return;
    // the end of a request is where client and scheduler meet again: ops of the next request wait for their grants even if
    // the scheduler needs a moment to start polling (see g_gave_up_in_pause)
    g_gave_up_in_pause[idx].store(0, std::memory_order_relaxed);
    if (it < 0 || it >= sh.request_status_len[idx]) {
        fprintf(stderr, "orion: block(%d) outside the %d requests announced for client %d\n", it, sh.request_status_len[idx], idx);
        return;
    }
    std::atomic<uint8_t>* st = sh.request_status[idx];
    const bool hp = idx == sh.num_clients - 1;
    uint32_t spins = 0;
    sh.rings[idx].blocked_on.store((int64_t)it + 1, std::memory_order_release);
    int64_t t0 = 0;
    while (!st[it].load(std::memory_order_acquire)) {
        if (!sh.active.load(std::memory_order_acquire)) break;
        ORION_PAUSE();
        ++spins;
        if (!hp && (spins & 0x3ff) == 0) sched_yield();
        if ((spins & 0xfffff) == 0) {
            int64_t now = mono_ms();
            if (!t0) t0 = now;
            if (now - t0 > 4 * gate_timeout_ms()) {
                fprintf(stderr, "orion: client %d gave up waiting for request %d to complete\n", idx, it);
                sh.wait_timeouts.fetch_add(1);
                break;
            }
        }
    }
    sh.rings[idx].blocked_on.store(0, std::memory_order_release);
}

// Cooperative stop: true once the scheduler asked this client to finish; the
// acknowledgement lets the scheduler count the client as done (intercept_temp.cpp:132-141).
bool stop() {
    orion_shared& sh = g_shared;
    int idx = client_index_of_thread();
    if (idx < 0) return false;
    bool res = sh.client_stop[idx].load(std::memory_order_acquire) != 0;
    if (res) sh.client_stop_ack[idx].store(1, std::memory_order_release);
    return res;
}

// Queue one op of the given record type without any CUDA call behind it: the hook
// for first-class ops and for host-only tests.  Returns the client index, -1 when
// the calling thread is not a registered client.
int orion_capture_op(int type) {
    Gate g;
    if (!gate_begin(&g, type, nullptr, 0)) return -1;
    gate_end(&g);
    return g.idx;
}

int orion_capture_client_index(void) { return client_index_of_thread(); }

void* orion_capture_client_stream(int idx) {
    if (idx < 0 || idx >= g_shared.num_clients) return nullptr;
    return g_shared.client_stream[idx];
}

// Register the calling thread as (a helper thread of) client `idx`; used for
// threads the scheduler could not know at setup time.
int orion_capture_register_thread(int idx) {
    orion_shared& sh = g_shared;
    if (idx < 0 || idx >= sh.num_clients) return -1;
    int tid = my_tid();
    for (int i = sh.num_clients + 1; i < ORION_MAX_THREADS; i++) {
        int32_t expect = 0;
        if (sh.thread_ids[i].load() == tid || sh.thread_ids[i].compare_exchange_strong(expect, tid)) {
            sh.thread_client[i].store(idx);
            sh.epoch.fetch_add(1);
            return 0;
        }
    }
    return -1;
}

// A kernel library declares `func` (the host-side handle its launches pass to cudaLaunchKernel) elastic:
// its result does not depend on gridDim.x, and it keeps `ctas_per_sm` CTAs resident per SM.  Under a grant
// that carries an SM quota q the launch interposers cut its grid to q * ctas_per_sm CTAs.
int orion_capture_mark_elastic(const void* func, int ctas_per_sm) {
    if (!func || ctas_per_sm <= 0) return -1;
    const uintptr_t f = (uintptr_t)func;
    unsigned h = elastic_hash(f);
    for (int probe = 0; probe < kElasticSlots; probe++, h = (h + 1) % kElasticSlots) {
        uintptr_t cur = g_elastic_func[h].load(std::memory_order_acquire);
        if (cur == f) {
            g_elastic_factor[h].store(ctas_per_sm, std::memory_order_release);
            return 0;
        }
        if (cur == 0) {
            uintptr_t expect = 0;
            if (g_elastic_func[h].compare_exchange_strong(expect, f, std::memory_order_acq_rel) || expect == f) {
                g_elastic_factor[h].store(ctas_per_sm, std::memory_order_release);
                return 0;
            }
        }
    }
    return -1;   // table full
}

// SM quota the scheduler would grant the calling client at this moment (0: whole device, or not a client).
int orion_capture_quota_hint(void) {
    int idx = client_index_of_thread();
    if (idx < 0) return 0;
    return g_shared.quota_hint[idx].load(std::memory_order_relaxed);
}

// SM quota carried by the latest grant of the calling thread (0: none).
int orion_capture_last_quota(void) { return tls_last_quota; }

// What the launch interposers would make of a grid of `grid_x` blocks of `func` under an SM quota of `num_ctas`.
unsigned orion_capture_clamp_grid(const void* func, unsigned grid_x, int num_ctas) { return clamp_grid(func, grid_x, num_ctas); }

unsigned long long orion_capture_clamped_launches(void) { return g_shared.clamped_launches.load(); }

unsigned long long orion_capture_count(int type) {
    if (type < 0) return g_shared.passthrough.load();
    return g_shared.captured[type & 31].load();
}

// Every intercepted call of a record type, whether it was scheduled or passed through.
unsigned long long orion_capture_seen(int type) { return g_shared.seen[type & 31].load(); }

}  // extern "C"
