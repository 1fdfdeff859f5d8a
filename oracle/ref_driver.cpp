// TEST INFRASTRUCTURE — not part of the product.
//
// ref_replay: drives the *reference's own* scheduler (its scheduler_eval.cpp and
// utils_sched.cpp, compiled unmodified into oracle/_ref/scheduler_eval.so by the
// Makefile beside this file) through an arrival script, with no GPU and no client
// threads, and writes the decision log that the product's policy must reproduce.
//
// How the reference is made deterministic.  Its polling loop touches the outside
// world only through symbols this executable supplies (it is linked -rdynamic and
// the scheduler library is loaded afterwards, so these definitions win):
//   * pthread_mutex_lock/unlock on the per-client queue mutexes
//       (scheduler_eval.cpp:285,301,392,419,463-466; utils_sched.cpp:114-116),
//   * cudaEventRecord / cudaEventQuery and the 19 launch entry points it dlsym()s
//       (utils_sched.cpp:159-237,520; scheduler_eval.cpp:338,346,399,405),
//   * std::chrono::system_clock::now (request latency, scheduler_eval.cpp:291,423),
//   * getpwuid (location of the capture library, scheduler_eval.cpp:554-558).
// Simulated clients push records into the reference's own std::queue objects from
// inside the mutex hook, i.e. exactly at the points where a real client could have
// won the mutex, and a per-stream FIFO timeline answers event queries.  The virtual
// clock advances one tick per non-pop queue lock, per submit and per event query.
// The same rules are implemented independently by the product's simulator; equal
// logs mean equal call sequences.
//
// Second mode, `ref_replay --observations <trace> <ref_dir>`: no simulation at all.  The trace
// (orion_b200/csrc/sched/observation.hpp) holds every answer the live scheduler got from its
// queues, events, clock and stop flags, and every op it released.  The same hooks hand those
// answers to the reference at the calls where it asks for them and compare what it releases,
// closes and stops with what the live run did, token by token.
#include <dlfcn.h>
#include <pwd.h>

#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "intercept_temp.h"   // the reference's record types (found through -I, never copied)

#include "../orion_b200/csrc/policy/arrival_script.hpp"   // script parser and log formatter only
#include "../orion_b200/csrc/policy/sim_env.hpp"

namespace {

struct SimClient {
    const orion::ScriptClient* sc = nullptr;
    int it = 0, k = 0;
    bool in_queue = false, waiting_done = false, stopped = false, stop_seen = false;
    int64_t next_push_at = 0, iter_earliest = 0;
    int iter_limit = 0;
};

struct Sim {
    bool active = false;
    int n = 0;
    int64_t now = 0;
    std::vector<SimClient> clients;
    std::vector<int64_t> busy;
    std::vector<int64_t> done_at;          // by event id
    bool pending = false;                  // a cudaEventRecord waits for its pop
    uintptr_t pend_event = 0, pend_stream = 0;
    orion::DecisionLog log;
    // the stand-in capture library's globals, as installed by the reference's setup()
    std::queue<func_record>** kqueues = nullptr;
    pthread_mutex_t** mutexes = nullptr;
    volatile bool** request_status = nullptr;
    volatile bool* client_stop = nullptr;
    volatile bool* client_stop_ack = nullptr;
    bool broken = false;
} g;

uintptr_t g_events = 0, g_streams = 0;
const int kEventsPerList = 30000;

const std::vector<orion::ScriptOp>& seq_of(const SimClient& c) {
    return (c.it == 0 && !c.sc->ops0.empty()) ? c.sc->ops0 : c.sc->ops;
}

void detect_stops() {
    for (int k = 0; k < g.n; k++) {
        if (!g.clients[k].stop_seen && g.client_stop[k]) {
            g.clients[k].stop_seen = true;
            g.log.add('X', g.now, k);
        }
    }
}

void touch(int i) {
    g.now += 1;
    SimClient& c = g.clients[i];
    if (!c.in_queue && !c.waiting_done && !c.stopped && c.it < c.iter_limit && c.it < c.sc->num_iters &&
        g.now >= c.next_push_at && !seq_of(c).empty()) {
        func_record r;
        memset((void*)&r, 0, sizeof r);
        r.type = (func_type)seq_of(c)[c.k].type;
        if (r.type == MEMCPY_RECORD) r.data.mrecord.async = true;
        if (r.type == MEMSET_RECORD) r.data.msetrecord.async = true;
        g.kqueues[i]->push(r);
        c.in_queue = true;
    }
}

void finalize_submit(int i) {
    g.now += 1;
    SimClient& c = g.clients[i];
    const std::vector<orion::ScriptOp>& ops = seq_of(c);
    if (!c.in_queue) {
        g.broken = true;
        return;
    }
    const orion::ScriptOp& op = ops[c.k];
    int stream = (int)g.pend_stream - 1;
    int64_t start = g.now > g.busy[stream] ? g.now : g.busy[stream];
    g.busy[stream] = start + op.dur;
    uintptr_t ev = g.pend_event - 1;
    g.done_at[ev] = g.busy[stream];
    g.log.add('S', g.now, i, op.type, stream, (int64_t)(ev / kEventsPerList), (int64_t)(ev % kEventsPerList));
    g.pending = false;
    c.in_queue = false;
    c.k += 1;
    if (c.k == (int)ops.size())
        c.waiting_done = true;
    else
        c.next_push_at = g.now + ops[c.k].gap;
}

void on_unlock(int i) {
    SimClient& c = g.clients[i];
    if (c.waiting_done && g.request_status[i][c.it]) {
        g.log.add('D', g.now, i, c.it);
        int64_t prev = c.iter_earliest;
        int64_t gap = c.sc->gaps.empty() ? 0 : c.sc->gaps[(size_t)c.it];
        c.it += 1;
        c.k = 0;
        c.waiting_done = false;
        if (g.client_stop[i]) {
            g.client_stop_ack[i] = true;
            c.stopped = true;
        } else {
            int64_t e = g.now + c.sc->think;
            c.iter_earliest = e > prev + gap ? e : prev + gap;
            const std::vector<orion::ScriptOp>& ops = seq_of(c);
            c.next_push_at = c.iter_earliest + (ops.empty() ? 0 : ops[0].gap);
        }
    }
}


// ------------------------------------------------------------------ observation mode
struct ObsTok {
    char kind;
    int a, b, c, d, e;
    int64_t t;
};
struct ObsLine {
    uint64_t rep;
    std::vector<ObsTok> toks;
};
struct Obs {
    bool on = false, truncated = false;
    const std::vector<ObsLine>* lines = nullptr;
    size_t line = 0, tok = 0;
    uint64_t rep = 0;
    uint64_t decisions = 0, closed = 0, queries = 0, tokens = 0, polls = 0;
    int64_t last_t = 0;
    std::vector<int> it;            // requests closed per client
    std::vector<int> max_it;        // length of the reference's request_status rows
    std::vector<char> stop_told;    // X tokens seen
    FILE* json_out = nullptr;
    int phase = 0;
} o;

[[noreturn]] void obs_finish(bool matched, const char* why) {
    fprintf(o.json_out,
            "{\"impl\": \"reference\", \"mode\": \"observations\", \"matched\": %s, \"truncated\": %s, \"decisions\": %llu, "
            "\"requests_closed\": %llu, \"queries\": %llu, \"polls\": %llu, \"phase\": %d, \"detail\": \"%s\"}\n",
            matched ? "true" : "false", o.truncated ? "true" : "false", (unsigned long long)o.decisions,
            (unsigned long long)o.closed, (unsigned long long)o.queries, (unsigned long long)o.polls, o.phase, why);
    fflush(o.json_out);
    _exit(matched ? 0 : 3);
}

const ObsTok* obs_cur() {
    while (o.line < o.lines->size()) {
        const ObsLine& l = (*o.lines)[o.line];
        if (o.tok < l.toks.size()) return &l.toks[o.tok];
        o.tok = 0;
        o.polls++;
        if (++o.rep >= l.rep) {
            o.rep = 0;
            o.line++;
        }
    }
    return nullptr;
}
void obs_advance() {
    o.tok++;
    o.tokens++;
}
// Tokens no call of the reference stands for: the stop-acknowledgement mask (the reference reads its flag from
// memory) and a stop request made while the client's lock is already held.
const ObsTok* obs_next(const char* who) {
    while (true) {
        const ObsTok* t = obs_cur();
        if (!t) {
            if (o.truncated) obs_finish(true, "the trace ends here (recording limit); every decision up to it agrees");
            static char msg[128];
            snprintf(msg, sizeof msg, "the reference made a call (%s) the live run did not make", who);
            obs_finish(false, msg);
        }
        if (t->kind == 'K') {
            for (int i = 0; i < g.n; i++) g.client_stop_ack[i] = (t->a >> i) & 1;
            obs_advance();
        } else if (t->kind == 'X' && t->b == 1) {
            o.stop_told[t->a] = 1;
            obs_advance();
        } else if (t->kind == 'B') {
            obs_finish(true, "the live run closed an iteration early (profile longer than the op stream); compared up to there");
        } else {
            return t;
        }
    }
}
[[noreturn]] void obs_mismatch(const char* what, const ObsTok* t, int a, int b, int c, int d, int e) {
    static char msg[256];
    snprintf(msg, sizeof msg, "%s: reference %d:%d:%d:%d:%d, live token %c%d:%d:%d:%d:%d", what, a, b, c, d, e, t->kind, t->a, t->b,
             t->c, t->d, t->e);
    obs_finish(false, msg);
}

void obs_lock(int i) {
    if (g.pending) {   // the pop that follows a launch: this is the decision
        int type = (int)g.kqueues[i]->front().type;
        int stream = (int)g.pend_stream - 1;
        uintptr_t ev = g.pend_event - 1;
        int evl = (int)(ev / kEventsPerList), evs = (int)(ev % kEventsPerList);
        const ObsTok* t = obs_next("release");
        if (t->kind != 'S' || t->a != i || t->b != type || t->c != stream || t->d != evl || t->e != evs)
            obs_mismatch("release", t, i, type, stream, evl, evs);
        obs_advance();
        o.decisions++;
        g.pending = false;
        return;
    }
    const ObsTok* t = obs_next("queue lock");
    if ((t->kind != 'P' && t->kind != 'L' && t->kind != 'X') || t->a != i) obs_mismatch("queue lock", t, i, 0, 0, 0, 0);
    if (t->kind == 'P') {
        std::queue<func_record>* q = g.kqueues[i];
        if (t->b >= 0) {
            if (q->empty()) {
                func_record r;
                memset((void*)&r, 0, sizeof r);
                r.type = (func_type)t->b;
                if (r.type == MEMCPY_RECORD) r.data.mrecord.async = true;
                if (r.type == MEMSET_RECORD) r.data.msetrecord.async = true;
                q->push(r);
            } else if ((int)q->front().type != t->b) {
                obs_mismatch("queue head", t, i, (int)q->front().type, 0, 0, 0);
            }
        } else if (!q->empty()) {
            obs_mismatch("queue should be empty", t, i, (int)q->front().type, 0, 0, 0);
        }
    } else if (t->kind == 'X') {
        o.stop_told[i] = 1;
    }
    obs_advance();
}

void obs_unlock(int i) {
    if (o.it[i] < o.max_it[i] && g.request_status[i][o.it[i]]) {
        const ObsTok* t = obs_next("request closed");
        if (t->kind != 'D' || t->a != i || t->b != o.it[i]) obs_mismatch("request closed", t, i, o.it[i], 0, 0, 0);
        obs_advance();
        o.it[i] += 1;
        o.closed++;
    }
}

bool obs_query(uintptr_t ev) {
    int evl = (int)(ev / kEventsPerList), evs = (int)(ev % kEventsPerList);
    const ObsTok* t = obs_next("event query");
    if (t->kind != 'Q' || t->a != evl || t->b != evs) obs_mismatch("event query", t, evl, evs, 0, 0, 0);
    bool done = t->c != 0;
    obs_advance();
    o.queries++;
    return done;
}

int64_t obs_now() {
    const ObsTok* t = obs_cur();
    if (t && t->kind == 'T') {
        o.last_t = t->t;
        obs_advance();
    }
    return o.last_t;
}

int client_of(pthread_mutex_t* m) {
    if (!g.active) return -1;
    for (int i = 0; i < g.n; i++)
        if (g.mutexes[i] == m) return i;
    return -1;
}

typedef int (*mutex_fn)(pthread_mutex_t*);
mutex_fn real_lock = nullptr, real_unlock = nullptr;

}  // namespace

// ------------------------------------------------------------------ interposed libc / libstdc++
extern "C" int pthread_mutex_lock(pthread_mutex_t* m) {
    int i = client_of(m);
    if (i < 0) {
        if (!real_lock) real_lock = (mutex_fn)dlsym(RTLD_NEXT, "pthread_mutex_lock");
        return real_lock(m);
    }
    if (o.on) {
        obs_lock(i);
        return 0;
    }
    detect_stops();
    if (g.pending)
        finalize_submit(i);
    else
        touch(i);
    return 0;
}

extern "C" int pthread_mutex_unlock(pthread_mutex_t* m) {
    int i = client_of(m);
    if (i < 0) {
        if (!real_unlock) real_unlock = (mutex_fn)dlsym(RTLD_NEXT, "pthread_mutex_unlock");
        return real_unlock(m);
    }
    if (o.on) {
        obs_unlock(i);
        return 0;
    }
    detect_stops();
    on_unlock(i);
    return 0;
}

static char g_home[8192];
static char g_home_base[4096];
extern "C" struct passwd* getpwuid(uid_t) {
    static struct passwd pw;
    strcpy(g_home, g_home_base);   // the reference strcat()s onto this buffer
    pw.pw_dir = g_home;
    pw.pw_name = (char*)"oracle";
    return &pw;
}

namespace std {
namespace chrono {
inline namespace _V2 {
system_clock::time_point system_clock::now() noexcept {
    if (o.on) return time_point(duration(obs_now() * 1000));
    return time_point(duration(g.now * 1000));   // 1 tick = 1 us; duration is ns
}
}  // namespace _V2
}  // namespace chrono
}  // namespace std

// ------------------------------------------------------------------ fake CUDA runtime / cuDNN / cuBLAS
extern "C" {
cudaError_t cudaDeviceGetStreamPriorityRange(int* least, int* greatest) {
    *least = 0;
    *greatest = -5;
    return cudaSuccess;
}
cudaError_t cudaStreamCreateWithPriority(cudaStream_t* s, unsigned int, int) {
    *s = (cudaStream_t)(++g_streams);
    return cudaSuccess;
}
cudaError_t cudaEventCreateWithFlags(cudaEvent_t* e, unsigned int) {
    *e = (cudaEvent_t)(++g_events);
    return cudaSuccess;
}
cudaError_t cudaEventRecord(cudaEvent_t e, cudaStream_t s) {
    g.pending = true;
    g.pend_event = (uintptr_t)e;
    g.pend_stream = (uintptr_t)s;
    return cudaSuccess;
}
cudaError_t cudaEventQuery(cudaEvent_t e) {
    if (o.on) return obs_query((uintptr_t)e - 1) ? cudaSuccess : cudaErrorNotReady;
    detect_stops();
    g.now += 1;
    uintptr_t ev = (uintptr_t)e - 1;
    bool done = g.now >= g.done_at[ev];
    g.log.add('Q', g.now, (int64_t)(ev / kEventsPerList), (int64_t)(ev % kEventsPerList), done ? 1 : 0);
    return done ? cudaSuccess : cudaErrorNotReady;
}
const char* cudaGetErrorString(cudaError_t) { return "fake"; }
cudnnStatus_t cudnnSetStream(cudnnHandle_t, cudaStream_t) { return CUDNN_STATUS_SUCCESS; }
cublasStatus_t cublasSetStream_v2(cublasHandle_t, cudaStream_t) { return CUBLAS_STATUS_SUCCESS; }

// The 19 launch entry points the reference dlsym()s live in fakecuda.cpp (a file
// without CUDA headers, so that variadic stubs do not clash with the real prototypes).
}

// ------------------------------------------------------------------ driver
typedef void* (*sched_init_fn)();
typedef void (*setup_fn)(void*, int, int*, char**, char**, int*, int*, bool*, bool);
typedef void (*setup_change_fn)(void*, int, char*, int);
typedef void* (*schedule_fn)(void*, int, bool, int, bool, int, bool, bool, int, int, int);

struct Ref {
    void* shim = nullptr;
    sched_init_fn sched_init = nullptr;
    setup_fn setup = nullptr;
    setup_change_fn setup_change = nullptr;
    schedule_fn schedule = nullptr;
    int* max_sms = nullptr;
};

static bool load_ref(const std::string& ref_dir, Ref& r) {
    void* sched_lib = dlopen((ref_dir + "/scheduler_eval.so").c_str(), RTLD_NOW | RTLD_GLOBAL);
    if (!sched_lib) {
        fprintf(stderr, "ref_replay: %s\n", dlerror());
        return false;
    }
    r.shim = dlopen((ref_dir + "/home/orion/src/cuda_capture/libinttemp.so").c_str(), RTLD_NOW | RTLD_GLOBAL);
    if (!r.shim) {
        fprintf(stderr, "ref_replay: %s\n", dlerror());
        return false;
    }
    r.sched_init = (sched_init_fn)dlsym(sched_lib, "sched_init");
    r.setup = (setup_fn)dlsym(sched_lib, "setup");
    r.setup_change = (setup_change_fn)dlsym(sched_lib, "setup_change");
    r.schedule = (schedule_fn)dlsym(sched_lib, "schedule");
    r.max_sms = (int*)dlsym(sched_lib, "max_sms");
    if (!r.sched_init || !r.setup || !r.setup_change || !r.schedule || !r.max_sms) {
        fprintf(stderr, "ref_replay: scheduler_eval.so lacks an expected symbol\n");
        return false;
    }
    return true;
}

static void bind_shim_globals(void* shim) {
    g.kqueues = *(std::queue<func_record>***)dlsym(shim, "kqueues");
    g.mutexes = *(pthread_mutex_t***)dlsym(shim, "mutexes");
    g.request_status = *(volatile bool***)dlsym(shim, "client_request_status");
    g.client_stop = *(volatile bool**)dlsym(shim, "client_stop");
    g.client_stop_ack = *(volatile bool**)dlsym(shim, "client_stop_ack");
}

// ---- observation mode: the trace file and its replay -------------------------------------------------
struct ObsCommand {
    enum Kind { PHASE, SETUP_CHANGE } kind;
    int args[7] = {0, 0, 0, 0, 0, 0, 0};   // phase: warmup, warmup_iters, reef, seq, depth, hp_limit, update_start
    std::vector<ObsLine> lines;
    int client = 0, num_kernels = 0;
    std::string file;
};

static bool parse_tokens(std::istringstream& in, std::vector<ObsTok>& out) {
    std::string w;
    while (in >> w) {
        ObsTok t{w[0], 0, 0, 0, 0, 0, 0};
        const char* p = w.c_str() + 1;
        if (t.kind == 'T') {
            t.t = strtoll(p, nullptr, 10);
        } else {
            int* f[5] = {&t.a, &t.b, &t.c, &t.d, &t.e};
            for (int k = 0; k < 5 && *p; k++) {
                char* end = nullptr;
                *f[k] = (int)strtol(p, &end, 10);
                p = (*end == ':') ? end + 1 : end;
            }
        }
        if (!strchr("PQTKBSLDX", t.kind)) return false;
        out.push_back(t);
    }
    return true;
}

static int run_observations(const std::string& trace, const std::string& ref_dir) {
    std::ifstream in(trace);
    if (!in.is_open()) {
        fprintf(stderr, "ref_replay: cannot open %s\n", trace.c_str());
        return 1;
    }
    const size_t slash = trace.find_last_of('/');
    const std::string trace_dir = slash == std::string::npos ? "." : trace.substr(0, slash);
    auto rel = [&](const std::string& p) { return (!p.empty() && p[0] == '/') ? p : trace_dir + "/" + p; };   // as the product's loader
    int max_sms = 80, reef_streams = 0, n = 0;
    std::vector<int> num_kernels, num_iters, trains;
    std::vector<std::string> profiles;
    std::vector<ObsCommand> cmds;
    bool truncated = false;
    std::string line, key;
    while (std::getline(in, line)) {
        std::istringstream ls(line);
        if (!(ls >> key)) continue;
        if (key == "orion_observations") continue;
        if (key == "max_sms") {
            std::string k2;
            ls >> max_sms >> k2 >> reef_streams;
        } else if (key == "nclients") {
            ls >> n;
            num_kernels.assign(n, 0);
            num_iters.assign(n, 0);
            trains.assign(n, 0);
            profiles.assign(n, "");
        } else if (key == "client") {
            int i;
            std::string k;
            ls >> i;
            if (i < 0 || i >= n) return 1;
            ls >> k >> trains[i] >> k >> num_iters[i] >> k >> profiles[i] >> num_kernels[i];
            profiles[i] = rel(profiles[i]);
        } else if (key == "phase") {
            ObsCommand c;
            c.kind = ObsCommand::PHASE;
            for (int k = 0; k < 7; k++) ls >> c.args[k];
            cmds.push_back(c);
        } else if (key == "p") {
            if (cmds.empty() || cmds.back().kind != ObsCommand::PHASE) return 1;
            ObsLine l;
            ls >> l.rep;
            if (!parse_tokens(ls, l.toks)) {
                fprintf(stderr, "ref_replay: unknown token in %s\n", trace.c_str());
                return 1;
            }
            if (!l.toks.empty() && l.rep > 0) cmds.back().lines.push_back(l);
        } else if (key == "setup_change") {
            ObsCommand c;
            c.kind = ObsCommand::SETUP_CHANGE;
            ls >> c.client >> c.file >> c.num_kernels;
            c.file = rel(c.file);
            cmds.push_back(c);
        } else if (key == "truncated") {
            truncated = true;
        } else if (key == "endphase" || key == "reset") {
            // `reset` only clears counters that are already zero between phases
        } else {
            fprintf(stderr, "ref_replay: unknown line '%s' in %s\n", key.c_str(), trace.c_str());
            return 1;
        }
    }
    if (n < 1 || cmds.empty()) {
        fprintf(stderr, "ref_replay: %s holds no phase\n", trace.c_str());
        return 1;
    }
    snprintf(g_home_base, sizeof g_home_base, "%s/home", ref_dir.c_str());
    o.json_out = fdopen(dup(1), "w");
    if (!freopen("/dev/null", "w", stdout)) return 1;
    Ref ref;
    if (!load_ref(ref_dir, ref)) return 1;
    *ref.max_sms = max_sms;

    std::vector<int> tids(n);
    std::vector<char*> models(n), files(n);
    bool* train = new bool[n];
    for (int i = 0; i < n; i++) {
        tids[i] = 100000 + i;
        models[i] = (char*)"model";
        files[i] = (char*)profiles[i].c_str();
        train[i] = trains[i] != 0;
    }
    g.n = n;
    void* sched = ref.sched_init();
    ref.setup(sched, n, tids.data(), models.data(), files.data(), num_kernels.data(), num_iters.data(), train, reef_streams != 0);
    bind_shim_globals(ref.shim);
    g.active = true;
    o.on = true;
    o.truncated = truncated;
    o.it.assign(n, 0);
    o.max_it = num_iters;
    o.stop_told.assign(n, 0);
    for (size_t c = 0; c < cmds.size(); c++) {
        ObsCommand& cmd = cmds[c];
        if (cmd.kind == ObsCommand::SETUP_CHANGE) {
            ref.setup_change(sched, cmd.client, (char*)cmd.file.c_str(), cmd.num_kernels);
            continue;
        }
        o.lines = &cmd.lines;
        o.line = o.tok = 0;
        o.rep = 0;
        ref.schedule(sched, n, true, 0, cmd.args[0] != 0, cmd.args[1], cmd.args[2] != 0, cmd.args[3] != 0, cmd.args[4], cmd.args[5],
                     cmd.args[6]);
        // the reference came back by itself: it must have used up the phase's tokens
        while (const ObsTok* t = obs_cur()) {
            if (t->kind == 'K' || (t->kind == 'X' && t->b == 1)) {
                if (t->kind == 'X') o.stop_told[t->a] = 1;
                obs_advance();
                continue;
            }
            if (o.truncated) break;
            obs_mismatch("the reference ended the phase, the live run went on", t, 0, 0, 0, 0, 0);
        }
        for (int k = 0; k < n; k++)
            if ((g.client_stop[k] ? 1 : 0) != o.stop_told[k]) {
                ObsTok x{'X', k, 0, 0, 0, 0, 0};
                obs_mismatch("stop request", &x, k, g.client_stop[k] ? 1 : 0, 0, 0, 0);
            }
        o.phase++;
    }
    obs_finish(true, "every release, closed request and stop request of the live run is the reference's");
}

int main(int argc, char** argv) {
    if (argc >= 4 && std::string(argv[1]) == "--observations") return run_observations(argv[2], argv[3]);
    if (argc < 4) {
        fprintf(stderr, "usage: ref_replay <script> <ref_dir> <log|-> [--quiet]\n       ref_replay --observations <trace> <ref_dir>\n");
        return 64;
    }
    std::string ref_dir = argv[2];
    std::string log_path = argv[3];
    orion::ArrivalScript s;
    try {
        s = orion::load_script(argv[1]);
    } catch (const std::exception& e) {
        fprintf(stderr, "ref_replay: %s\n", e.what());
        return 1;
    }
    int n = (int)s.clients.size();
    snprintf(g_home_base, sizeof g_home_base, "%s/home", ref_dir.c_str());

    // The reference prints progress on stdout; keep stdout for the JSON line only.
    FILE* json_out = fdopen(dup(1), "w");
    if (!freopen("/dev/null", "w", stdout)) return 1;

    Ref ref;
    if (!load_ref(ref_dir, ref)) return 1;
    sched_init_fn sched_init = ref.sched_init;
    setup_fn setup = ref.setup;
    setup_change_fn setup_change = ref.setup_change;
    schedule_fn schedule = ref.schedule;
    void* shim = ref.shim;
    *ref.max_sms = s.max_sms;

    std::vector<int> tids(n), num_kernels(n), num_iters(n);
    std::vector<char*> models(n), files(n);
    bool* train = new bool[n];
    for (int i = 0; i < n; i++) {
        tids[i] = 100000 + i;
        num_kernels[i] = s.clients[i].num_kernels;
        num_iters[i] = s.clients[i].num_iters;
        models[i] = (char*)"model";
        files[i] = (char*)s.clients[i].profile.c_str();
        train[i] = s.clients[i].train;
    }
    g.n = n;
    g.clients.resize(n);
    g.busy.assign(n, 0);
    g.done_at.assign((size_t)n * kEventsPerList, 0);
    for (int i = 0; i < n; i++) {
        g.clients[i].sc = &s.clients[i];
        g.clients[i].next_push_at = seq_of(g.clients[i]).empty() ? 0 : seq_of(g.clients[i])[0].gap;
    }

    bool reef = s.algo == "reef", seq = s.algo == "sequential";
    void* sched = sched_init();
    setup(sched, n, tids.data(), models.data(), files.data(), num_kernels.data(), num_iters.data(), train, reef);
    if (g_events != (uintptr_t)n * kEventsPerList || g_streams != (uintptr_t)n) {
        fprintf(stderr, "ref_replay: setup created %lu events and %lu streams, expected %d and %d\n",
                (unsigned long)g_events, (unsigned long)g_streams, n * kEventsPerList, n);
        return 1;
    }
    bind_shim_globals(shim);
    g.active = true;

    double secs = 0;
    for (size_t p = 0; p < s.phases.size(); p++) {
        for (SimClient& c : g.clients) c.iter_limit = s.phases[p].warmup ? s.phases[p].warmup_iters : c.sc->num_iters;
        auto t0 = std::chrono::steady_clock::now();
        schedule(sched, n, true, 0, s.phases[p].warmup, s.phases[p].warmup_iters, reef, seq, s.depth, s.hp_limit,
                 s.update_start);
        auto t1 = std::chrono::steady_clock::now();
        secs += std::chrono::duration<double>(t1 - t0).count();
        detect_stops();
        g.log.add('E', (int64_t)p);
        if (g.broken) {
            fprintf(stderr, "ref_replay: script inconsistent with the scheduler's pops\n");
            return 2;
        }
        if (p == 0) {
            for (int i = 0; i < n; i++)
                if (!s.clients[i].profile2.empty())
                    setup_change(sched, i, (char*)s.clients[i].profile2.c_str(), s.clients[i].num_kernels2);
        }
    }
    g.active = false;
    if (log_path != "-" && !g.log.write(log_path)) {
        fprintf(stderr, "ref_replay: cannot write %s\n", log_path.c_str());
        return 1;
    }
    size_t decisions = g.log.count('S');
    fprintf(json_out,
            "{\"impl\": \"reference\", \"decisions\": %zu, \"queries\": %zu, \"iters_done\": %zu, \"seconds\": %.6f, "
            "\"decisions_per_s\": %.1f, \"log_fnv1a\": \"%016llx\"}\n",
            decisions, g.log.count('Q'), g.log.count('D'), secs, decisions / secs,
            (unsigned long long)g.log.fnv1a());
    fflush(json_out);
    _exit(0);   // the reference leaks its scheduler state by design; skip static destructors
}
