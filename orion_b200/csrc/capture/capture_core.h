// Internal interface between the capture core and the interposers.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "../policy/op_types.h"
#include "capture_state.h"

namespace orion_capture {

struct LaunchInfo {       // filled by the kernel-launch interposers for the profile recorder
    const void* func;
    unsigned grid[3], block[3];
    size_t shared_mem;
};

struct Gate {
    int idx;        // client index; -2 = unscheduled call that is being profiled
    uint64_t seq;
    void* stream;   // stream to launch on (the caller's, or the client's scheduler stream)
    void* event;    // event to record behind the op
    int num_ctas;   // SM quota of the grant (0 = no limit)
    int type;
    uint64_t tag;
    const LaunchInfo* launch;
    void* prof_start;
};

// Returns false when the calling thread is not a scheduled client (pass through).
// Otherwise queues a record, waits for the scheduler's grant and fills `g`.
bool gate_begin(Gate* g, int type, void* user_stream, uint64_t tag);
// Records the granted event on the granted stream and retires the record.
void gate_end(Gate* g);

// Grid width to launch `func` with under a grant of `num_ctas` SMs: kernels registered as elastic (their
// blocks walk the work with a gridDim.x stride, so any grid width gives the same result) are cut to
// num_ctas x their CTAs-per-SM factor; every other kernel keeps its grid.
unsigned clamp_grid(const void* func, unsigned grid_x, int num_ctas);

int client_index_of_thread();
int client_index_of_stream(void* stream);

// cudaEventRecord of the real runtime (resolved lazily; a no-op when no CUDA
// runtime is loaded, which is the case in host-only tests).
void real_event_record(void* event, void* stream);

// Profile recorder (profile_recorder.cpp): active when ORION_PROFILE_OUT is set.
bool profile_enabled();
void profile_begin(Gate* g);
void profile_end(Gate* g);
void profile_mark_iteration(int it);

}  // namespace orion_capture
