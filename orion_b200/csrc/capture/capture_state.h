// Shared state between the capture library (client side) and the scheduler.
//
// The reference shares nine raw globals — thread-id table, one std::queue plus
// pthread mutex per client, request-status matrix, stop flags
// (src/cuda_capture/intercept_temp.cpp:8-19) — which its scheduler allocates
// through dlsym (src/scheduler/scheduler_eval.cpp:572-657).  Here the same
// information lives in one versioned block owned by the capture library, and each
// client queue is a lock-free single-producer/single-consumer ring.
//
// Protocol for one captured call (the client thread runs steps 1,3,4; the
// scheduler thread runs step 2):
//   1. push:    ring[tail % CAP] = {type,...}; tail.store(tail+1, release)
//   2. grant:   the policy picks the head; the scheduler writes the stream, the
//               event to record behind the op and the SM quota of the grant (the
//               number of CTAs a persistent kernel may occupy) and publishes
//               granted = head+1
//   3. launch:  the client thread, which has been spinning on `granted`, performs
//               the real CUDA/cuBLAS/cuDNN call itself on the granted stream and
//               records the granted event — so launch cost is paid on the client's
//               core, not on the single scheduler core, and real return codes reach
//               the caller
//   4. retire:  submitted.store(head+1, release); the scheduler joins on this
//               before it queries an event of that client.
// `granted` doubles as the consumer index of the ring and is advanced by
// compare-and-swap: between two schedule() calls nobody polls, and a memory
// operation queued then (for example the read-back of a result right after
// block(it) returned) grants itself instead of waiting for the next phase.
// The client never has more than one call between push and retire, which is the
// reference's behaviour (its interposers spin until the queue is empty,
// src/cuda_capture/utils_interc.cpp:53-64); the ring capacity leaves room for a
// deeper pipeline later.
#pragma once
#include <stdint.h>

#include <atomic>

#define ORION_CAPTURE_ABI_VERSION 2
#define ORION_MAX_CLIENTS 16
#define ORION_RING_CAP 64
#define ORION_MAX_THREADS (2 * ORION_MAX_CLIENTS + 1)

struct orion_record {
    int32_t type;          // orion_rec_type
    int32_t flags;
    uint64_t tag;          // kernel function pointer or library handle, for traces/profiles
};

struct alignas(64) orion_grant {
    void* stream;          // cudaStream_t to launch on
    void* event;           // cudaEvent_t to record behind the op (may be null)
    int num_ctas;          // SM quota of this grant: a kernel whose grid is elastic (see orion_capture_mark_elastic)
                           // is launched with at most this many CTAs per resident-CTA slot; 0 = no limit
};

struct alignas(64) orion_ring {
    // written by the client
    alignas(64) std::atomic<uint64_t> tail;
    alignas(64) std::atomic<uint64_t> submitted;
    std::atomic<int64_t> blocked_on;         // request index + 1 while the client sits in block(it), else 0
    // written by the scheduler
    alignas(64) std::atomic<uint64_t> granted;
    orion_grant grant;
    alignas(64) orion_record recs[ORION_RING_CAP];
};

struct orion_shared {
    int abi_version;
    std::atomic<int> active;                 // scheduler attached: interposers queue instead of passing through
    std::atomic<int> polling;                // the scheduler is inside schedule(); outside it, queued memory
                                             // operations grant themselves (they bypass every policy rule anyway)
    int num_clients;
    std::atomic<int> epoch;                  // bumped whenever the thread table changes
    std::atomic<int32_t> thread_ids[ORION_MAX_THREADS];   // [0,N): clients, [N]: scheduler, rest: helper threads
    std::atomic<int32_t> thread_client[ORION_MAX_THREADS];
    void* client_stream[ORION_MAX_CLIENTS];  // stream the scheduler created for each client
    orion_ring rings[ORION_MAX_CLIENTS];
    std::atomic<uint8_t>* request_status[ORION_MAX_CLIENTS];   // [max_iters] per client
    int request_status_len[ORION_MAX_CLIENTS];
    std::atomic<uint8_t> client_stop[ORION_MAX_CLIENTS];
    std::atomic<uint8_t> client_stop_ack[ORION_MAX_CLIENTS];
    std::atomic<uint8_t> affinity_set[ORION_MAX_THREADS];
    int pin_threads;                         // 0: leave affinity alone
    int core_offset;                         // first core for client 0 (reference: 1, or 4 with two clients)
    int n_cores;                             // > 0: pin inside this list instead (the process's own affinity mask, so
    int core_list[256];                      //      that replicas with disjoint masks stay disjoint): scheduler thread
                                             //      on core_list[0], client i on core_list[(1 + i) % n_cores]
    // SM quota the scheduler would grant client i right now (a hint for planning a launch before it is queued;
    // the quota that binds is the one in the grant); 0 = the whole device
    std::atomic<int> quota_hint[ORION_MAX_CLIENTS];
    std::atomic<uint64_t> clamped_launches;  // kernel launches whose grid was cut to the granted quota
    // statistics
    std::atomic<uint64_t> captured[32];      // per record type
    std::atomic<uint64_t> passthrough;       // intercepted calls from unknown threads
    std::atomic<uint64_t> seen[32];          // every intercepted call, scheduled or not, per record type
    std::atomic<uint64_t> wait_timeouts;     // bounded waits that expired
};

extern "C" {
// The one accessor the scheduler needs; everything else hangs off the block.
orion_shared* orion_capture_shared(void);
}
