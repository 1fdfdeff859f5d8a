// orion_replay: run an arrival script through the policy core in virtual time.
//
//   orion_replay <script> [--log <file>] [--repeat <n>]
//   orion_replay --observations <trace>
//
// The second form feeds an observation trace of a live run (observation.hpp) to the policy core: the recorded queue heads,
// event answers, clock reads and stop acknowledgements go in, and every release, lock, closed request and stop request the
// core makes is compared with the recorded one.
//
// Prints one JSON line with the decision count, the FNV-1a hash of the decision
// log and the wall time of the policy loop (decisions per second on one core).
// The phase sequence mirrors PyScheduler.run_scheduler (src/scheduler_frontend.py:68-94):
// after the first phase the clients that name a second profile get it installed,
// as setup_change does (src/scheduler/scheduler_eval.cpp:528-540).
#include <chrono>
#include <cstdio>
#include <cstring>
#include <string>

#include "../policy/arrival_script.hpp"
#include "../policy/policy.hpp"
#include "../policy/sim_env.hpp"
#include "observation.hpp"

using namespace orion;

static int run_once(const ArrivalScript& s, DecisionLog* out, PolicyStats* stats, double* secs) {
    int n = (int)s.clients.size();
    std::vector<int> num_kernels(n), num_iters(n);
    PolicyCore core;
    core.max_sms = s.max_sms;
    core.op_info.resize(n);
    for (int i = 0; i < n; i++) {
        num_kernels[i] = s.clients[i].num_kernels;
        num_iters[i] = s.clients[i].num_iters;
        load_profile(s.clients[i].profile, core.op_info[i]);
        core.max_sms_clients.push_back(max_sm_used(core.op_info[i]));
        core.is_train.push_back(s.clients[i].train);
    }
    core.init(n, num_kernels.data(), num_iters.data());
    SimEnv env(s);
    PhaseArgs a;
    a.reef = s.algo == "reef";
    a.seq = s.algo == "sequential";
    a.depth = s.depth;
    a.hp_limit = s.hp_limit;
    a.update_start = s.update_start;
    auto t0 = std::chrono::steady_clock::now();
    for (size_t p = 0; p < s.phases.size(); p++) {
        a.warmup = s.phases[p].warmup;
        a.warmup_iters = s.phases[p].warmup_iters;
        env.begin_phase(s.phases[p]);
        core.run_phase(env, a);
        env.end_phase((int)p);
        if (core.error || env.broken) return 2;
        if (p == 0) {
            for (int i = 0; i < n; i++) {
                if (s.clients[i].profile2.empty()) continue;
                core.op_info[i].clear();
                load_profile(s.clients[i].profile2, core.op_info[i]);
                core.max_sms_clients[i] = max_sm_used(core.op_info[i]);
                num_kernels[i] = s.clients[i].num_kernels2;
            }
        }
    }
    auto t1 = std::chrono::steady_clock::now();
    *secs = std::chrono::duration<double>(t1 - t0).count();
    *stats = core.stats;
    *out = std::move(env.log);
    return 0;
}

static int run_observations(const char* path) {
    ObsTrace t = load_obs_trace(path);
    const int n = t.n;
    PolicyCore core;
    core.max_sms = t.max_sms;
    core.op_info.resize(n);
    for (int i = 0; i < n; i++) {
        load_profile(t.profiles[i], core.op_info[i]);
        core.max_sms_clients.push_back(max_sm_used(core.op_info[i]));
        core.is_train.push_back(t.train[i] != 0);
    }
    core.init(n, t.num_kernels.data(), t.num_iters.data());
    core.max_events = 30000;
    ObsReplayEnv env;
    bool matched = true, cut = false;
    std::string detail = "every release, closed request and stop request of the live run is reproduced";
    int phase = 0;
    try {
        for (ObsTraceCmd& c : t.cmds) {
            if (!c.is_phase) {
                core.op_info[c.client].clear();
                load_profile(c.file, core.op_info[c.client]);
                core.max_sms_clients[c.client] = max_sm_used(core.op_info[c.client]);
                t.num_kernels[c.client] = c.num_kernels;
                continue;
            }
            PhaseArgs a;
            a.warmup = c.args[0] != 0;
            a.warmup_iters = c.args[1];
            a.reef = c.args[2] != 0;
            a.seq = c.args[3] != 0;
            a.depth = c.args[4];
            a.hp_limit = c.args[5];
            a.update_start = c.args[6];
            env.begin(&c.lines);
            core.run_phase(env, a);
            if (core.error) throw ObsMismatch{false, "the policy core stopped on an unsupported record or an event overflow"};
            if (!env.drained() && !t.truncated) throw ObsMismatch{false, "the policy core ended the phase, the live run went on"};
            phase++;
        }
    } catch (const ObsMismatch& m) {
        if (m.exhausted && t.truncated) {
            cut = true;
            detail = "the trace ends here (recording limit); every decision up to it is reproduced";
        } else {
            matched = false;
            detail = m.detail;
        }
    }
    printf("{\"impl\": \"orion_b200\", \"mode\": \"observations\", \"matched\": %s, \"truncated\": %s, \"decisions\": %llu, "
           "\"requests_closed\": %llu, \"polls\": %llu, \"phase\": %d, \"detail\": \"%s\"}\n",
           matched ? "true" : "false", (t.truncated || cut) ? "true" : "false", (unsigned long long)env.decisions,
           (unsigned long long)env.closed, (unsigned long long)env.polls, phase, detail.c_str());
    return matched ? 0 : 3;
}

int main(int argc, char** argv) {
    if (argc >= 3 && !strcmp(argv[1], "--observations")) {
        try {
            return run_observations(argv[2]);
        } catch (const std::exception& e) {
            fprintf(stderr, "orion_replay: %s\n", e.what());
            return 1;
        }
    }
    if (argc < 2) {
        fprintf(stderr, "usage: orion_replay <script> [--log file] [--repeat n]\n       orion_replay --observations <trace>\n");
        return 64;
    }
    std::string log_path;
    int repeat = 1;
    for (int i = 2; i < argc; i++) {
        if (!strcmp(argv[i], "--log") && i + 1 < argc) log_path = argv[++i];
        else if (!strcmp(argv[i], "--repeat") && i + 1 < argc) repeat = atoi(argv[++i]);
    }
    try {
        ArrivalScript s = load_script(argv[1]);
        DecisionLog log;
        PolicyStats st;
        double best = 1e30, secs = 0;
        for (int r = 0; r < repeat; r++) {
            int rc = run_once(s, &log, &st, &secs);
            if (rc) {
                fprintf(stderr, "orion_replay: policy aborted (unsupported record or inconsistent script)\n");
                return rc;
            }
            if (secs < best) best = secs;
        }
        if (!log_path.empty() && !log.write(log_path)) {
            fprintf(stderr, "orion_replay: cannot write %s\n", log_path.c_str());
            return 1;
        }
        size_t decisions = log.count('S');
        printf("{\"impl\": \"orion_b200\", \"decisions\": %zu, \"queries\": %zu, \"iters_done\": %zu, \"polls\": %llu, "
               "\"be_rejects\": %llu, \"seconds\": %.6f, \"decisions_per_s\": %.1f, \"log_fnv1a\": \"%016llx\"}\n",
               decisions, log.count('Q'), log.count('D'), (unsigned long long)st.polls,
               (unsigned long long)st.be_rejects, best, decisions / best, (unsigned long long)log.fnv1a());
    } catch (const std::exception& e) {
        fprintf(stderr, "orion_replay: %s\n", e.what());
        return 1;
    }
    return 0;
}
