/* liborion_sched.so — C ABI of the scheduler library.
 *
 * The first six entry points are the ones the reference's Python front binds with
 * ctypes (reference src/scheduler_frontend.py:15,60,72-91 calling the extern "C"
 * block of reference src/scheduler/scheduler_eval.cpp:489-676); names, argument
 * order and meaning are kept so that a `cdll.LoadLibrary` of this library can take
 * the place of `scheduler_eval.so`.  The orion_sched_* entry points are additions.
 *
 * Threading: all calls come from one thread; `schedule` blocks until every client
 * finished the phase.  Errors: like the reference, failures are reported on stderr
 * (an unreadable profile or an unsupported record type aborts the process,
 * reference scheduler_eval.cpp:504 and utils_sched.cpp:514-516).
 */
#ifndef ORION_SCHED_H
#define ORION_SCHED_H
#include <stdbool.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct Scheduler Scheduler;

/* reference scheduler_eval.cpp:491-495 */
Scheduler* sched_init(void);

/* reference scheduler_eval.cpp:542-660.  tids: native thread ids of the client
 * threads; files: per-client profile files (Name,Profile,Memory_footprint,SM_usage,
 * Duration); num_kernels / num_iters: BORROWED and kept for the whole run (the
 * reference keeps the pointers too, :608-609) — setup_change writes into
 * num_kernels.  The high-priority client is the last one. */
void setup(Scheduler* s, int num_clients, int* tids, char** models, char** files, int* num_kernels, int* num_iters,
           bool* train, bool reef);

/* reference scheduler_eval.cpp:528-540: install another profile for one client. */
void setup_change(Scheduler* s, int client_id, char* file, int num_kernels);

/* reference scheduler_eval.cpp:663-670.  profile_mode must be true; `reef_depth`
 * carries DUR_THRESHOLD (ns) when the Orion policy runs. */
void* schedule(Scheduler* s, int num_clients, bool profile_mode, int iter, bool warmup, int warmup_iters, bool reef, bool seq,
               int reef_depth, int hp_limit, int update_start);

/* reference scheduler_eval.cpp:672-675 */
void* reset(Scheduler* s, int num_clients);

/* populate_kernel_info (reference scheduler_eval.cpp:498-526) takes a C++ vector
 * and is therefore exported with C++ linkage only; C callers use this variant:
 * parses a profile file, copies up to `cap` rows, returns the row count or -1. */
int orion_load_profile(const char* path, int* profile, int* sm_used, float* duration, int cap);

/* ---- additions: no counterpart in the reference ---- */
void* orion_sched_client_stream(Scheduler* s, int idx);   /* cudaStream_t created for client idx */
void orion_sched_shutdown(Scheduler* s);                  /* detach: queued clients run unscheduled */
/* out[0..8] = polls, hp_submits, be_submits, be_rejects, event queries, join timeouts,
 * max_sms, green-context best-effort SMs, forced iteration ends */
void orion_sched_stats(Scheduler* s, unsigned long long* out, int n);
int orion_sched_durations(Scheduler* s, int idx, float* out_ms, int cap);   /* scheduler-side latency samples */
int orion_sched_cur_iter(Scheduler* s, int idx);

#ifdef __cplusplus
}
#endif
#endif
