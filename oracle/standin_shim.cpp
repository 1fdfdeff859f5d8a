// TEST INFRASTRUCTURE — not part of the product.
//
// Stand-in for the capture library that the reference scheduler dlopen()s in
// setup() (src/scheduler/scheduler_eval.cpp:554-658).  The scheduler only needs
// the nine global pointer variables of src/cuda_capture/intercept_temp.cpp:8-19
// to exist; it allocates what they point to itself.  No interposer lives here:
// under the oracle there are no client threads.
#include <sys/types.h>
volatile pid_t* thread_ids;
void** kqueues;
void** mutexes;
int* func_indexes;
int* num_total_clients;
volatile bool** client_request_status;
volatile bool* client_stop;
volatile bool* client_stop_ack;
volatile bool* affinity_set;
