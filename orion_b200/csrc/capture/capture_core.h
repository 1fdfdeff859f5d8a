// Internal interface between the capture core and the interposers.
#pragma once
#include <stdint.h>

#include "../policy/op_types.h"
#include "capture_state.h"

namespace orion_capture {

struct Gate {
    int idx;
    uint64_t seq;
    void* stream;   // stream to launch on (the caller's, or the client's scheduler stream)
    void* event;    // event to record behind the op
};

// Returns false when the calling thread is not a scheduled client (pass through).
// Otherwise queues a record, waits for the scheduler's grant and fills `g`.
bool gate_begin(Gate* g, int type, void* user_stream, uint64_t tag);
// Records the granted event on the granted stream and retires the record.
void gate_end(Gate* g);

int client_index_of_thread();
int client_index_of_stream(void* stream);

// cudaEventRecord of the real runtime (resolved lazily; a no-op when no CUDA
// runtime is loaded, which is the case in host-only tests).
void real_event_record(void* event, void* stream);

}  // namespace orion_capture
