// liborion_sched.so — the scheduler library behind src/scheduler_frontend.py.
//
// Exports the reference's C entry points with the reference's signatures
// (src/scheduler/scheduler_eval.cpp:489-676): sched_init, setup, setup_change,
// schedule, reset, populate_kernel_info.  The polling loop is PolicyCore (a
// decision-for-decision restatement of the reference policy) driven by LiveEnv:
// lock-free ring heads from the capture library, real CUDA streams and events.
//
// Differences from the reference that do not change decisions:
//   * the granted op is launched by the client thread that captured it (see
//     capture_state.h), so HP and BE launch costs overlap instead of serialising on
//     the scheduler thread; the scheduler joins a client's outstanding launch before
//     it queries that client's events;
//   * the CUDA runtime is bound at run time, so the library also loads on a machine
//     without a GPU (ORION_FAKE_GPU=1 swaps in an "everything completes at once"
//     device for host-only tests);
//   * optional: the best-effort stream can live in a green context with a fixed SM
//     quota (ORION_BE_SM_QUOTA), which turns the profile-trusted SM budget into a
//     hardware partition;
//   * optional: the run can be recorded as an arrival script (ORION_RECORD_SCRIPT)
//     for replay through orion_replay and through the reference scheduler, and as an
//     observation trace (ORION_RECORD_OBS, observation.hpp): every answer the policy got
//     and every decision it took, for a check of the live decisions against the reference.
#include <dlfcn.h>
#include <pthread.h>
#include <sched.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <chrono>
#include <string>
#include <vector>

#include "../capture/capture_state.h"
#include "../policy/policy.hpp"
#include "green_ctx.hpp"
#include "observation.hpp"

#if defined(__x86_64__)
#include <immintrin.h>
#define ORION_PAUSE() _mm_pause()
#else
#define ORION_PAUSE() ((void)0)
#endif

namespace {

using orion::OpInfo;

// ---------------------------------------------------------------- CUDA runtime binding
typedef int (*fn_prio_range)(int*, int*);
typedef int (*fn_stream_create)(void**, unsigned, int);
typedef int (*fn_event_create)(void**, unsigned);
typedef int (*fn_event_query)(void*);
typedef int (*fn_get_device)(int*);
typedef int (*fn_dev_attr)(int*, int, int);

struct CudaApi {
    bool fake = false;
    fn_prio_range prio_range = nullptr;
    fn_stream_create stream_create = nullptr;
    fn_event_create event_create = nullptr;
    fn_event_query event_query = nullptr;
    fn_get_device get_device = nullptr;
    fn_dev_attr dev_attr = nullptr;
    std::string error;

    bool bind() {
        const char* fk = getenv("ORION_FAKE_GPU");
        if (fk && atoi(fk)) {
            fake = true;
            return true;
        }
        void* h = dlopen("libcudart.so.12", RTLD_NOW | RTLD_NOLOAD);
        if (!h) h = dlopen("libcudart.so.12", RTLD_NOW);
        if (!h) h = dlopen("/usr/local/cuda/lib64/libcudart.so.12", RTLD_NOW);
        if (!h) {
            error = "libcudart.so.12 is not loadable (set ORION_FAKE_GPU=1 for host-only runs)";
            return false;
        }
        prio_range = (fn_prio_range)dlsym(h, "cudaDeviceGetStreamPriorityRange");
        stream_create = (fn_stream_create)dlsym(h, "cudaStreamCreateWithPriority");
        event_create = (fn_event_create)dlsym(h, "cudaEventCreateWithFlags");
        event_query = (fn_event_query)dlsym(h, "cudaEventQuery");
        get_device = (fn_get_device)dlsym(h, "cudaGetDevice");
        dev_attr = (fn_dev_attr)dlsym(h, "cudaDeviceGetAttribute");
        if (!prio_range || !stream_create || !event_create || !event_query || !get_device || !dev_attr) {
            error = "libcudart.so.12 lacks an expected symbol";
            return false;
        }
        return true;
    }
};

constexpr int kEventsPerClient = 30000;   // utils_sched.cpp:150
constexpr unsigned kStreamNonBlocking = 1;
constexpr unsigned kEventDisableTiming = 2;

inline int64_t wall_us() {
    return std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

struct RecordedOp {
    int type;
    int64_t gap_us;
};

// ---------------------------------------------------------------- live environment
struct LiveEnv {
    orion_shared* sh = nullptr;
    CudaApi* api = nullptr;
    int n = 0;
    std::vector<void*> streams;
    std::vector<std::vector<void*>> events;
    std::vector<std::vector<uint64_t>> ev_seq;          // grant sequence behind each event slot
    std::vector<std::vector<int>> ev_owner;             // client whose launch records the slot
    uint64_t join_timeouts = 0;
    // SM quota of best-effort grants (execution side; no decision depends on it)
    orion::PolicyCore* core = nullptr;
    bool quota_on = false;
    int quota_reserve = 0;    // SMs left free for the high-priority client while it has no request in flight
    int quota_floor = 8;      // a best-effort grant never goes below this
    int quota_gran = 8;       // SM-partition granularity of the device
    uint64_t quota_grants = 0, quota_ctas_sum = 0;
    uint32_t idle_polls = 0;
    // An inference client's events are only ever queried for the last compute op of a request (iteration end,
    // policy.hpp; the update-phase rule needs a training high-priority client).  Its other ops are granted without an
    // event, so nothing sits between two of its kernels in the stream and a kernel may begin while its predecessor
    // drains (programmatic dependent launch).  Queries and their answers are unchanged.
    bool skip_inner_events = true;
    // recording (arrival-script abstraction of the run)
    bool recording = false;
    std::vector<int64_t> last_pop_us;
    std::vector<std::vector<RecordedOp>> cur_iter_ops;
    std::vector<std::vector<std::vector<RecordedOp>>> rec_iters;   // per client, per iteration
    std::vector<std::vector<int64_t>> iter_start_us;

    int peek(int i) {
        orion_ring& r = sh->rings[i];
        uint64_t head = r.granted.load(std::memory_order_acquire);
        uint64_t tail = r.tail.load(std::memory_order_acquire);
        if (tail <= head) return -1;
        return r.recs[head % ORION_RING_CAP].type;
    }
    int64_t now_us() { return wall_us(); }
    // SM quota a best-effort client is granted right now: the device's SMs minus the SM need of the
    // high-priority op in flight (the value the reference stores at scheduler_eval.cpp:317 and never uses),
    // or minus a fixed reserve while no high-priority request is in flight; rounded down to the partition
    // granularity.  0 = no limit (the high-priority client, a single client, or the feature switched off).
    int quota_for(int i) const {
        if (!quota_on || n < 2 || i == n - 1 || !core) return 0;
        const int hp = n - 1;
        const int max_sms = core->max_sms;
        const bool hp_in_flight = core->seen[hp] > 0;
        int need = hp_in_flight ? core->hp_sm_need : quota_reserve;
        if (need <= 0) return 0;
        int q = (max_sms - need) / quota_gran * quota_gran;
        if (q < quota_floor) q = quota_floor;
        return q >= max_sms ? 0 : q;
    }
    void poll_end(bool progressed) {
        if (quota_on)
            for (int i = 0; i + 1 < n; i++) sh->quota_hint[i].store(quota_for(i), std::memory_order_relaxed);
        // Nothing moved for a while: ease off the core in short bursts so that a client thread spinning
        // on the sibling hardware thread gets the issue slots (a poll is then a fraction of a microsecond late).
        if (progressed) {
            idle_polls = 0;
        } else if (++idle_polls > 64) {
            for (int k = 0; k < 8; k++) ORION_PAUSE();
        }
    }
    void submit(int i, int type, int stream, int evl, int evs) {
        orion_ring& r = sh->rings[i];
        if (recording) {
            int64_t t = wall_us();
            if (cur_iter_ops[i].empty()) iter_start_us[i].push_back(t);
            cur_iter_ops[i].push_back(RecordedOp{type, last_pop_us[i] ? t - last_pop_us[i] : 0});
            last_pop_us[i] = t;
        }
        uint64_t head = r.granted.load(std::memory_order_acquire);
        r.grant.stream = streams[stream];
        const bool inner_op_of_inference_request = skip_inner_events && core && evl == i && !core->is_train[i] &&
                                                   (orion_is_memop(type) || core->seen[i] + 1 < core->num_kernels[i]);
        r.grant.event = inner_op_of_inference_request ? nullptr : events[evl][evs];
        const int q = orion_is_memop(type) ? 0 : quota_for(i);
        r.grant.num_ctas = q;
        if (q > 0) {
            quota_grants++;
            quota_ctas_sum += (uint64_t)q;
        }
        ev_seq[evl][evs] = head + 1;
        ev_owner[evl][evs] = i;
        // Fails only if the client granted itself a memory operation in the instant
        // this phase started; that record is then already on its way.
        r.granted.compare_exchange_strong(head, head + 1, std::memory_order_acq_rel);
    }
    bool query(int evl, int evs) {
        // The event is recorded by the client thread right after its launch; make sure
        // that has happened before asking the device.
        int owner = ev_owner[evl][evs];
        if (owner >= 0) {
            orion_ring& r = sh->rings[owner];
            uint64_t need = ev_seq[evl][evs];
            if (r.submitted.load(std::memory_order_acquire) < need) {
                int64_t t0 = wall_us();
                while (r.submitted.load(std::memory_order_acquire) < need) {
                    if (wall_us() - t0 > 2000000) {   // a client died between grant and launch
                        join_timeouts++;
                        sh->wait_timeouts.fetch_add(1);
                        return false;
                    }
                }
            }
        }
        if (api->fake) return true;
        return api->event_query(events[evl][evs]) == 0;
    }
    void iter_lock(int) {}   // nothing to lock: a ring is not peeked while its iteration drains
    void iter_done(int i, int iter) {
        if (recording) {
            rec_iters[i].push_back(cur_iter_ops[i]);
            cur_iter_ops[i].clear();
        }
        if (iter >= 0 && iter < sh->request_status_len[i]) sh->request_status[i][iter].store(1, std::memory_order_release);
    }
    void stop(int k, bool) { sh->client_stop[k].store(1, std::memory_order_release); }
    bool stop_ack(int i) { return sh->client_stop_ack[i].load(std::memory_order_acquire) != 0; }
    bool client_blocked(int i, int iter) {
        orion_ring& r = sh->rings[i];
        uint64_t head = r.granted.load(std::memory_order_acquire);
        return r.blocked_on.load(std::memory_order_acquire) == (int64_t)iter + 1 &&
               r.tail.load(std::memory_order_acquire) == head && r.submitted.load(std::memory_order_acquire) == head;
    }
};

}  // namespace

// ---------------------------------------------------------------- the scheduler object
struct Scheduler {
    orion::PolicyCore core;
    LiveEnv env;
    CudaApi api;
    orion::GreenCtx green;
    orion_shared* sh = nullptr;
    void* capture_lib = nullptr;
    int num_clients = 0;
    bool ready = false;
    std::vector<std::string> profile_paths;
    std::string record_path;
    orion::ObsRecorder obs;
    int phases_run = 0;
};

static orion_shared* find_capture(Scheduler* s) {
    typedef orion_shared* (*acc_fn)(void);
    acc_fn acc = (acc_fn)dlsym(RTLD_DEFAULT, "orion_capture_shared");
    if (!acc) {
        // Not preloaded: load it from $ORION_CAPTURE_LIB or from beside this library.
        std::string path;
        if (const char* e = getenv("ORION_CAPTURE_LIB")) path = e;
        if (path.empty()) {
            Dl_info info;
            if (dladdr((void*)&find_capture, &info) && info.dli_fname) {
                path = info.dli_fname;
                size_t slash = path.find_last_of('/');
                path = (slash == std::string::npos ? std::string(".") : path.substr(0, slash)) + "/liborion_capture.so";
            }
        }
        s->capture_lib = dlopen(path.c_str(), RTLD_NOW | RTLD_GLOBAL);
        if (!s->capture_lib) {
            fprintf(stderr, "orion: cannot load the capture library: %s\n", dlerror());
            return nullptr;
        }
        acc = (acc_fn)dlsym(s->capture_lib, "orion_capture_shared");
    }
    return acc ? acc() : nullptr;
}

static void write_recorded_script(Scheduler* s, const orion::PhaseArgs& a);

// The policy indexes a client's profile with its op counter up to num_kernels - 1 (policy.hpp, as the
// reference does at scheduler_eval.cpp:306,330): a profile with fewer rows than that, or none, would make
// it decide on memory past the vector.  The reference has the same hole; here the run ends with a message.
static void check_profile_rows(const char* where, int client, const char* file, int rows, int num_kernels) {
    if (rows < 1 || num_kernels < 1 || num_kernels > rows) {
        fprintf(stderr, "orion: %s: client %d announces %d kernels per iteration but its profile %s has %d rows\n", where, client,
                num_kernels, file ? file : "(null)", rows);
        abort();
    }
}

extern "C" {

Scheduler* sched_init() { return new Scheduler(); }

// Same contract as the reference's loader; exposed for tools.  Returns the row count, -1 on error.
int populate_kernel_info(char* kernel_info_file, std::vector<OpInfo>& ops) {
    try {
        orion::load_profile(kernel_info_file, ops);
    } catch (const std::exception& e) {
        fprintf(stderr, "%s\n", e.what());
        return -1;
    }
    return (int)ops.size();
}

// C-friendly variant: parses a profile and copies up to `cap` rows of (profile, sm_used, duration).
int orion_load_profile(const char* path, int* profile, int* sm_used, float* duration, int cap) {
    std::vector<OpInfo> ops;
    try {
        orion::load_profile(path, ops);
    } catch (const std::exception& e) {
        fprintf(stderr, "%s\n", e.what());
        return -1;
    }
    for (int i = 0; i < (int)ops.size() && i < cap; i++) {
        if (profile) profile[i] = ops[i].profile;
        if (sm_used) sm_used[i] = ops[i].sm_used;
        if (duration) duration[i] = ops[i].duration;
    }
    return (int)ops.size();
}

void setup_change(Scheduler* s, int client_id, char* file, int num_kernels) {
    if (!s || client_id < 0 || client_id >= s->num_clients) return;
    s->core.op_info[client_id].clear();
    try {
        orion::load_profile(file, s->core.op_info[client_id]);
    } catch (const std::exception& e) {
        fprintf(stderr, "%s\n", e.what());
        abort();   // the reference asserts on an unreadable profile
    }
    check_profile_rows("setup_change", client_id, file, (int)s->core.op_info[client_id].size(), num_kernels);
    s->core.max_sms_clients[client_id] = orion::max_sm_used(s->core.op_info[client_id]);
    s->core.num_kernels[client_id] = num_kernels;   // written into the caller's array, like the reference
    s->profile_paths[client_id] = file;
    if (s->obs.f) s->obs.raw("setup_change " + std::to_string(client_id) + " " + file + " " + std::to_string(num_kernels));
}

void setup(Scheduler* s, int num_clients, int* tids, char** models, char** files, int* num_kernels, int* num_iters, bool* train,
           bool reef) {
    (void)models;
    if (!s || num_clients < 1 || num_clients > ORION_MAX_CLIENTS) {
        fprintf(stderr, "orion: setup: between 1 and %d clients are supported\n", ORION_MAX_CLIENTS);
        return;
    }
    s->sh = find_capture(s);
    if (!s->sh || s->sh->abi_version != ORION_CAPTURE_ABI_VERSION) {
        fprintf(stderr, "orion: capture library missing or of another ABI version\n");
        return;
    }
    if (!s->api.bind()) {
        fprintf(stderr, "orion: %s\n", s->api.error.c_str());
        return;
    }
    orion_shared* sh = s->sh;
    s->num_clients = num_clients;

    // 1. thread table: clients, then this (scheduler) thread, then free helper slots
    sh->active.store(0);
    sh->polling.store(0);
    sh->num_clients = num_clients;
    for (int i = 0; i < ORION_MAX_THREADS; i++) {
        sh->thread_ids[i].store(0);
        sh->thread_client[i].store(-1);
        sh->affinity_set[i].store(0);
    }
    for (int i = 0; i < num_clients; i++) {
        sh->thread_ids[i].store(tids[i]);
        sh->thread_client[i].store(i);
    }
    sh->thread_ids[num_clients].store((int)syscall(SYS_gettid));
    sh->thread_client[num_clients].store(num_clients);
    const char* pin = getenv("ORION_PIN_THREADS");
    sh->pin_threads = pin ? atoi(pin) : 0;
    const char* off = getenv("ORION_CORE_OFFSET");
    sh->core_offset = off ? atoi(off) : (num_clients == 2 ? 4 : 1);   // reference offsets, utils_interc.cpp:37-41
    // ORION_PIN_THREADS=2: pin inside the cores this process may run on, so that replicas started with
    // disjoint affinity masks (one per GPU) never share a core: this scheduler thread takes the first core
    // of the mask, client i the (1 + i)-th; other threads (autograd workers) float inside the mask.
    sh->n_cores = 0;
    if (sh->pin_threads == 2) {
        cpu_set_t mask;
        CPU_ZERO(&mask);
        if (sched_getaffinity(0, sizeof(mask), &mask) == 0) {
            for (int c = 0; c < CPU_SETSIZE && sh->n_cores < 256; c++)
                if (CPU_ISSET(c, &mask)) sh->core_list[sh->n_cores++] = c;
        }
        if (sh->n_cores >= num_clients + 1) {
            cpu_set_t one;
            CPU_ZERO(&one);
            CPU_SET(sh->core_list[0], &one);
            if (sched_setaffinity(0, sizeof(one), &one) != 0) perror("orion: sched_setaffinity (scheduler thread)");
        } else {
            sh->n_cores = 0;      // too few cores to give every spinning thread its own: leave affinity alone
            sh->pin_threads = 0;
        }
    }

    // 2. profiles
    orion::PolicyCore& core = s->core;
    core = orion::PolicyCore();
    core.op_info.resize(num_clients);
    s->profile_paths.assign(num_clients, "");
    for (int i = 0; i < num_clients; i++) {
        try {
            orion::load_profile(files[i], core.op_info[i]);
        } catch (const std::exception& e) {
            fprintf(stderr, "%s\n", e.what());
            abort();
        }
        check_profile_rows("setup", i, files[i], (int)core.op_info[i].size(), num_kernels[i]);
        core.max_sms_clients.push_back(orion::max_sm_used(core.op_info[i]));
        core.is_train.push_back(train[i]);
        s->profile_paths[i] = files[i];
    }
    core.init(num_clients, num_kernels, num_iters);   // both arrays are borrowed and kept
    core.max_events = kEventsPerClient;

    // max_sms: the reference hard-codes 80 (V100); default to the device's SM count.
    int max_sms = 80;
    if (const char* e = getenv("ORION_MAX_SMS")) {
        max_sms = atoi(e);
    } else if (!s->api.fake) {
        int dev = 0, cnt = 0;
        if (s->api.get_device(&dev) == 0 && s->api.dev_attr(&cnt, 16 /*cudaDevAttrMultiProcessorCount*/, dev) == 0 && cnt > 0)
            max_sms = cnt;
    }
    core.max_sms = max_sms;

    // 3. queues and run-time control
    for (int i = 0; i < num_clients; i++) {
        orion_ring& r = sh->rings[i];
        r.tail.store(0);
        r.submitted.store(0);
        r.granted.store(0);
        r.blocked_on.store(0);
        delete[] sh->request_status[i];
        int len = num_iters[i] > 0 ? num_iters[i] : 0;
        sh->request_status[i] = new std::atomic<uint8_t>[(size_t)len + 1];
        for (int k = 0; k <= len; k++) sh->request_status[i][k].store(0);
        sh->request_status_len[i] = len;
        sh->client_stop[i].store(0);
        sh->client_stop_ack[i].store(0);
    }

    // 4. streams (best-effort: priority 0; high-priority client = last index: greatest
    //    priority unless REEF, utils_sched.cpp:119-144) and events
    LiveEnv& env = s->env;
    env = LiveEnv();
    env.sh = sh;
    env.api = &s->api;
    env.n = num_clients;
    env.streams.assign(num_clients, nullptr);
    env.events.assign(num_clients, {});
    env.ev_seq.assign(num_clients, std::vector<uint64_t>(kEventsPerClient, 0));
    env.ev_owner.assign(num_clients, std::vector<int>(kEventsPerClient, -1));
    env.core = &s->core;
    {   // SM quota carried by best-effort grants; ORION_SM_QUOTA=0 switches it off
        const char* q = getenv("ORION_SM_QUOTA");
        env.quota_on = !(q && q[0] == '0') && num_clients > 1;
        if (const char* e = getenv("ORION_HP_RESERVE_SMS")) env.quota_reserve = atoi(e);
        if (const char* e = getenv("ORION_BE_MIN_SMS")) env.quota_floor = atoi(e) > 0 ? atoi(e) : 8;
        for (int i = 0; i < ORION_MAX_CLIENTS; i++) sh->quota_hint[i].store(0);
    }
    int lp = 0, hp = 0;
    if (!s->api.fake) s->api.prio_range(&lp, &hp);
    int be_quota = 0;
    if (const char* e = getenv("ORION_BE_SM_QUOTA")) be_quota = atoi(e);
    if (be_quota > 0 && !s->api.fake && num_clients > 1) {
        if (!s->green.create(be_quota)) {
            fprintf(stderr, "orion: green-context partition unavailable (%s); using plain priority streams\n",
                    s->green.error.c_str());
            be_quota = 0;
        }
    }
    for (int i = 0; i < num_clients; i++) {
        const bool is_hp = i == num_clients - 1;
        const int prio = (is_hp && !reef) ? hp : 0;
        if (s->api.fake) {
            env.streams[i] = (void*)(uintptr_t)(0x1000 + i);
        } else if (be_quota > 0) {
            env.streams[i] = s->green.stream(is_hp ? 1 : 0, prio);
            if (!env.streams[i]) s->api.stream_create(&env.streams[i], kStreamNonBlocking, prio);
        } else {
            s->api.stream_create(&env.streams[i], kStreamNonBlocking, prio);
        }
        sh->client_stream[i] = env.streams[i];
        env.events[i].resize(kEventsPerClient);
        for (int j = 0; j < kEventsPerClient; j++) {
            if (s->api.fake)
                env.events[i][j] = nullptr;
            else
                s->api.event_create(&env.events[i][j], kEventDisableTiming);
        }
    }
    if (const char* e = getenv("ORION_RECORD_SCRIPT")) {
        s->record_path = e;
        env.recording = true;
        env.last_pop_us.assign(num_clients, 0);
        env.cur_iter_ops.assign(num_clients, {});
        env.rec_iters.assign(num_clients, {});
        env.iter_start_us.assign(num_clients, {});
    }
    if (const char* e = getenv("ORION_RECORD_OBS")) {
        uint64_t cap = 400000;   // distinct poll lines; a trace stops there and says so
        if (const char* c = getenv("ORION_RECORD_OBS_MAX_LINES")) cap = strtoull(c, nullptr, 10);
        s->obs.close();
        s->obs = orion::ObsRecorder();
        if (s->obs.open(e, cap)) {
            std::string h = "orion_observations 1\nmax_sms " + std::to_string(core.max_sms) + " reef " + (reef ? "1" : "0") +
                            "\nnclients " + std::to_string(num_clients);
            for (int i = 0; i < num_clients; i++)
                h += "\nclient " + std::to_string(i) + " train " + (train[i] ? "1" : "0") + " num_iters " +
                     std::to_string(num_iters[i]) + " profile " + files[i] + " " + std::to_string(num_kernels[i]);
            s->obs.raw(h);
        } else {
            fprintf(stderr, "orion: cannot write the observation trace %s\n", e);
        }
    }
    sh->epoch.fetch_add(1);
    sh->active.store(1, std::memory_order_release);
    s->ready = true;
}

void* schedule(Scheduler* s, int num_clients, bool profile_mode, int iter, bool warmup, int warmup_iters, bool reef, bool seq,
               int reef_depth, int hp_limit, int update_start) {
    (void)iter;
    if (!s || !s->ready || !profile_mode || num_clients != s->num_clients) return nullptr;
    orion::PhaseArgs a;
    a.warmup = warmup;
    a.warmup_iters = warmup_iters;
    a.reef = reef;
    a.seq = seq;
    a.depth = reef_depth;
    a.hp_limit = hp_limit;
    a.update_start = update_start;
    {
        const char* e = getenv("ORION_SKIP_INNER_EVENTS");
        s->env.skip_inner_events = !seq && !(e && e[0] == '0');   // the sequential policy shares one event list
    }
    s->sh->polling.store(1, std::memory_order_release);
    if (s->obs.on()) {
        char line[160];
        snprintf(line, sizeof line, "phase %d %d %d %d %d %d %d", warmup ? 1 : 0, warmup_iters, reef ? 1 : 0, seq ? 1 : 0, reef_depth,
                 hp_limit, update_start);
        s->obs.raw(line);
        orion::ObsEnv<LiveEnv> watched(s->env, s->obs, s->num_clients);
        watched.begin_phase();
        s->core.run_phase(watched, a);
        watched.end_phase();
        s->obs.raw("endphase");
        if (!warmup || s->obs.truncated) s->obs.close();
    } else {
        s->core.run_phase(s->env, a);
    }
    s->sh->polling.store(0, std::memory_order_release);
    s->phases_run++;
    if (s->core.error == 2) {
        fprintf(stderr, "orion: an iteration has more than %d compute ops, the number of events per client - ABORT\n",
                kEventsPerClient);
        abort();
    }
    if (s->core.error) {
        fprintf(stderr, "UNSUPPORTED OPERATION - ABORT\n");   // utils_sched.cpp:514-516
        abort();
    }
    if (!warmup && s->env.recording) write_recorded_script(s, a);
    return nullptr;
}

void* reset(Scheduler* s, int num_clients) {
    (void)num_clients;
    if (s) s->core.reset();
    if (s && s->obs.f) s->obs.raw("reset");
    return nullptr;
}

// ---- additions (not in the reference) ----

// Stream the scheduler created for client `idx`; the launcher runs the client under it.
void* orion_sched_client_stream(Scheduler* s, int idx) {
    if (!s || idx < 0 || idx >= s->num_clients) return nullptr;
    return s->env.streams[idx];
}

// Detach: interposers pass through again and any client spinning on a grant is released.
void orion_sched_shutdown(Scheduler* s) {
    if (s && s->sh) s->sh->active.store(0, std::memory_order_release);
}

// stats: [polls, hp_submits, be_submits, be_rejects, queries, join_timeouts, max_sms, green_be_sms, forced_iter_ends,
//         quota_grants (best-effort grants that carried an SM quota), quota_ctas_sum (sum of those quotas),
//         clamped_launches (kernel launches the capture library cut to their quota)]
void orion_sched_stats(Scheduler* s, unsigned long long* out, int n) {
    if (!s || !out) return;
    unsigned long long v[12] = {s->core.stats.polls,      s->core.stats.hp_submits, s->core.stats.be_submits,
                                s->core.stats.be_rejects, s->core.stats.queries,    s->env.join_timeouts,
                                (unsigned long long)s->core.max_sms, (unsigned long long)s->green.be_sms,
                                s->core.stats.forced_iter_ends, s->env.quota_grants, s->env.quota_ctas_sum,
                                s->sh ? s->sh->clamped_launches.load() : 0ull};
    for (int i = 0; i < n && i < 12; i++) out[i] = v[i];
}

// Latency samples (ms) the scheduler measured for client `idx` (scheduler_eval.cpp:423-426).
int orion_sched_durations(Scheduler* s, int idx, float* out, int cap) {
    if (!s || idx < 0 || idx >= s->num_clients) return -1;
    const std::vector<float>& d = s->core.client_durations[idx];
    for (int i = 0; i < (int)d.size() && i < cap; i++) out[i] = d[i];
    return (int)d.size();
}

int orion_sched_cur_iter(Scheduler* s, int idx) {
    if (!s || idx < 0 || idx >= s->num_clients) return -1;
    return s->core.cur_iters[idx];
}

}  // extern "C"

// Write the measured phase as an arrival script: per client the op types and host
// gaps of a representative steady-state iteration, device durations from the
// profile rows, and the observed request start distances.
static void write_recorded_script(Scheduler* s, const orion::PhaseArgs& a) {
    LiveEnv& env = s->env;
    FILE* f = fopen(s->record_path.c_str(), "w");
    if (!f) return;
    fprintf(f, "orion_script 1\nalgo %s\ndepth %d hp_limit %d update_start %d max_sms %d\nnclients %d\n",
            a.reef ? "reef" : (a.seq ? "sequential" : "orion"), a.depth, a.hp_limit, a.update_start, s->core.max_sms,
            s->num_clients);
    for (int i = 0; i < s->num_clients; i++) {
        const auto& iters = env.rec_iters[i];
        // steady state = the last complete iteration whose compute-op count matches the profile
        const std::vector<RecordedOp>* pick = nullptr;
        for (size_t k = iters.size(); k-- > 0;) {
            int compute = 0;
            for (const RecordedOp& o : iters[k]) compute += !orion_is_memop(o.type);
            if (compute == s->core.num_kernels[i]) {
                pick = &iters[k];
                break;
            }
        }
        int n_iters = (int)iters.size();
        if (const char* cap = getenv("ORION_RECORD_MAX_ITERS"))   // bound the length of the replay
            if (atoi(cap) > 0 && n_iters > atoi(cap)) n_iters = atoi(cap);
        if (n_iters < 12) n_iters = 12;
        fprintf(f, "client %d\n  train %d num_iters %d think 0\n  profile %s %d\n", i, s->core.is_train[i] ? 1 : 0, n_iters,
                s->profile_paths[i].c_str(), s->core.num_kernels[i]);
        fprintf(f, "  ops %d", pick ? (int)pick->size() : 0);
        if (pick) {
            size_t row = 0;
            for (const RecordedOp& o : *pick) {
                long dur = 0;
                if (!orion_is_memop(o.type) && row < s->core.op_info[i].size()) dur = (long)(s->core.op_info[i][row++].duration / 1000.0f);
                fprintf(f, " %d %ld %ld", orion_reference_type(o.type), (long)(o.gap_us < 0 ? 0 : o.gap_us), dur < 1 ? 1 : dur);
            }
        }
        fprintf(f, "\n");
        const auto& st = env.iter_start_us[i];
        if (!s->core.is_train[i] && st.size() > 1) {
            fprintf(f, "  gaps open");
            for (int k = 0; k < n_iters; k++) {
                long g = (k + 1 < (int)st.size()) ? (long)(st[k + 1] - st[k]) : 0;
                fprintf(f, " %ld", g < 0 ? 0 : g);
            }
            fprintf(f, "\n");
        } else {
            fprintf(f, "  gaps closed\n");
        }
        fprintf(f, "end\n");
    }
    fprintf(f, "phases 3 1 1 1 10 0 0\n");
    fclose(f);
}
