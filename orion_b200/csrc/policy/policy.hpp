// The co-location policy as a clock-free, CUDA-free step loop.
//
// `PolicyCore::run_phase` restates Scheduler::busy_wait_profile
// (src/scheduler/scheduler_eval.cpp:238-487) together with schedule_reef
// (:93-165) and schedule_sequential (:167-236).  Everything the reference
// touches outside its own counters — queue heads, stream launches, event
// queries, client mutexes, wall-clock reads, the stop flags — goes through an
// `Env` object, so the same code drives
//   * the live scheduler (ring-queue heads, real streams and events), and
//   * trace replay / the virtual-time simulator used for decision parity.
// The order of Env calls is part of the contract: it equals the order in which
// the reference locks client mutexes, launches, records and queries events.
//
// Env must provide:
//   int     peek(int client)            head record type of the client queue, -1 if empty
//                                       (the reference's lock / size() / front() / unlock)
//   int64_t now_us()                    clock for latency samples (microseconds)
//   void    submit(int client, int type, int stream, int ev_list, int ev_slot)
//                                       replay the head on stream `stream`, record event
//                                       (ev_list, ev_slot) behind it, pop the queue
//   bool    query(int ev_list, int ev_slot)   true when that event has completed
//   void    iter_lock(int client)       scheduler takes the client's queue lock and keeps it
//   void    iter_done(int client, int iter)   request `iter` complete: publish and unlock
//   void    stop(int client, bool locked)     ask a best-effort client to stop
//   bool    stop_ack(int client)        client acknowledged the stop
//   void    poll_end(bool progressed)   end of one pass of the loop; `progressed` = an op was released or an
//                                       iteration closed in it.  A hook for the live scheduler (publishing the SM
//                                       quota, easing off the core when nothing moves); replay environments ignore it.
//   bool    client_blocked(int client, int iter)
//                                       live runs only: the client already waits for request
//                                       `iter` to complete and has nothing queued.  If that
//                                       happens before the profile's op count was reached, the
//                                       profile is longer than the real op sequence and the
//                                       iteration is closed instead of deadlocking.  Replay
//                                       environments return false; the reference has no such
//                                       escape (it would hang).
//
// Quirks kept on purpose, because decisions must equal the reference's:
//   * `size` restarts at 0 every poll and only sums ops admitted in that poll;
//   * the HP op's SM need is stored but never read; HP inference => threshold = max_sms;
//   * `profiles[hp]` survives the HP op it came from;
//   * memory ops skip every rule, add their row's sm_used to `size` but not to `sum`;
//   * `sum` is a long that accumulates float durations through float arithmetic;
//   * the round-robin cursor only moves when a best-effort op is admitted;
//   * sequential mode releases only warm-up and malloc records (the reference's
//     own comment says it is unfinished).
#pragma once
#include <climits>
#include <cstdint>
#include <vector>

#include "op_types.h"
#include "profile_csv.hpp"

namespace orion {

enum Algo { ALGO_ORION = 0, ALGO_REEF = 1, ALGO_SEQUENTIAL = 2 };

struct PhaseArgs {
    bool warmup = false;
    int warmup_iters = 0;
    bool reef = false;
    bool seq = false;
    int depth = 1;          // DUR_THRESHOLD (orion) or queue depth (reef)
    int hp_limit = 1;
    int update_start = 1;
};

struct PolicyStats {
    uint64_t polls = 0;
    uint64_t hp_submits = 0;
    uint64_t be_submits = 0;
    uint64_t be_rejects = 0;      // a best-effort head was seen and not released in that poll
    uint64_t queries = 0;
    uint64_t forced_iter_ends = 0;   // iterations closed because the profile was longer than the op stream
};

class PolicyCore {
public:
    int max_sms = 80;                           // scheduler_eval.cpp:20 (V100); overridable
    int num_clients = 0;
    std::vector<std::vector<OpInfo>> op_info;   // one profile per client
    std::vector<int> max_sms_clients;
    std::vector<char> is_train;
    int* num_kernels = nullptr;                 // borrowed from the caller, like the reference
    int* max_iters = nullptr;                   // borrowed
    std::vector<int> seen, event_ids, cur_iters;
    std::vector<char> locked;
    std::vector<int64_t> client_starts, total_client_starts;
    std::vector<std::vector<char>> starts_set;
    std::vector<std::vector<float>> client_durations;   // ms per finished request
    int penalty = 0;                            // reef; survives across phases
    int error = 0;                              // 1 = unsupported record type seen, 2 = more compute ops in one
                                                // iteration than there are events per client
    int max_events = INT_MAX;                   // events per client list (the reference creates 30000 and never checks)
    uint64_t released = 0;                      // ops handed to Env::submit so far
    int hp_sm_need = 0;                         // SM need of the high-priority op released last: what the reference
                                                // stores in cur_sms[hp] (scheduler_eval.cpp:317) and never reads.  No
                                                // decision depends on it; the live scheduler sizes the SM quota of
                                                // best-effort grants with it.
    PolicyStats stats;

    void init(int n, int* kernels, int* iters) {
        num_clients = n;
        num_kernels = kernels;
        max_iters = iters;
        seen.assign(n, 0);
        event_ids.assign(n, 0);
        cur_iters.assign(n, 0);
        locked.assign(n, 0);
        client_starts.assign(n, 0);
        total_client_starts.assign(n, 0);
        starts_set.resize(n);
        for (int i = 0; i < n; i++) starts_set[i].assign((size_t)(iters[i] > 0 ? iters[i] : 0) + 1, 0);
        client_durations.assign(n, {});
    }

    // Scheduler::profile_reset (scheduler_eval.cpp:49-56)
    void reset() {
        for (int i = 0; i < num_clients; i++) seen[i] = 0;
    }

    template <class Env>
    void run_phase(Env& env, const PhaseArgs& a);

private:
    // schedule_kernel's bookkeeping (utils_sched.cpp:239-522): compute ops advance the
    // op counter of `idx` and the event cursor of list `evid`; memory ops advance neither.
    template <class Env>
    void submit(Env& env, int type, int stream, int idx, int evid) {
        if (orion_is_unsupported(type)) {
            error = 1;
            return;
        }
        int slot = event_ids[evid];   // the event pointer is taken before the increment
        if (slot >= max_events) {
            error = 2;
            return;
        }
        env.submit(idx, type, stream, evid, slot);
        released++;
        if (!orion_is_memop(type)) {
            event_ids[evid] += 1;
            seen[idx] += 1;
        }
    }

    template <class Env>
    void schedule_reef(Env& env, const std::vector<int>& heads, int depth);
    template <class Env>
    int schedule_sequential(Env& env, const std::vector<int>& heads, int start);
};

template <class Env>
void PolicyCore::schedule_reef(Env& env, const std::vector<int>& heads, int depth) {
    const int n = num_clients;
    if (n == 1) {
        if (heads[0] >= 0) submit(env, heads[0], 0, 0, 0);
        return;
    }
    const int hp = n - 1;
    for (int i = 0; i < n; i++) {
        if (heads[i] >= 0 &&
            (heads[i] == ORION_MALLOC_RECORD || cur_iters[i] <= 10 || cur_iters[hp] >= max_iters[hp])) {
            submit(env, heads[i], i, i, i);
            return;
        }
    }
    if (heads[hp] >= 0) {
        int hp_idx = seen[hp];
        submit(env, heads[hp], hp, hp, hp);
        const OpInfo& op1 = op_info[hp][hp_idx];
        for (int i = 0; i < hp; i++) {
            if (heads[i] < 0) continue;
            const OpInfo& op0 = op_info[i][seen[i]];
            if (op0.duration <= op1.duration && op0.sm_used >= op1.sm_used) {
                submit(env, heads[i], i, i, i);
                stats.be_submits++;
                return;
            }
        }
    } else {
        for (int i = 0; i < hp; i++)
            if (heads[i] >= 0) penalty += 1;
        if (penalty >= depth) {
            for (int i = 0; i < hp; i++)
                if (heads[i] >= 0) {
                    submit(env, heads[i], i, i, i);
                    stats.be_submits++;
                }
            penalty = 0;
        }
    }
}

template <class Env>
int PolicyCore::schedule_sequential(Env& env, const std::vector<int>& heads, int start) {
    const int n = num_clients;
    if (n == 1) {
        if (heads[0] >= 0) submit(env, heads[0], 0, 0, 0);
        return start;
    }
    const int hp = n - 1;
    if (heads[hp] >= 0) {
        // Only warm-up requests and malloc records are ever released here: the
        // "no other client active" branch can only clear the flag.
        bool go = (cur_iters[hp] <= 10) || (heads[hp] == ORION_MALLOC_RECORD);
        if (go) submit(env, heads[hp], 0, hp, 0);
    }
    int end = start + n;
    for (int t = start + 1; t < end; t++) {
        int i = t % (n - 1);
        if (heads[i] < 0) continue;
        bool go = cur_iters[i] <= 10 || heads[i] == ORION_MALLOC_RECORD;
        if (go) {
            submit(env, heads[i], 0, i, 0);
            start = t;
            break;
        }
    }
    return start;
}

template <class Env>
void PolicyCore::run_phase(Env& env, const PhaseArgs& a) {
    const int n = num_clients;
    const int hp = n - 1;
    const bool warmup = a.warmup, reef = a.reef, seq = a.seq;
    const int depth = a.depth;
    int update_start = a.update_start;

    std::vector<char> total_client_set(n, 0);
    std::vector<int> profiles(n, -1);
    std::vector<int> heads(n, -1);

    bool large_found = false;
    long sum = 0;    // durations of best-effort ops released since the last drain
    long size = 0;   // SM need of best-effort ops released in this poll
    int start = -1;

    int low_sms = 0;
    int high_sms = max_sms_clients[0];
    int sm_threshold = max_sms_clients[0] / 2;
    float hp_iter_duration = 0.0f;
    float hp_limit_float = (float)a.hp_limit;
    if (!is_train[hp]) {
        sm_threshold = max_sms;
        update_start = INT_MAX;
    }

    while (true) {
        stats.polls++;
        size = 0;
        const uint64_t released_before = released;
        bool closed_iter = false;
        for (int i = 0; i < n; i++) {
            heads[i] = -1;
            if (seen[i] == num_kernels[i]) continue;
            if (seen[i] > 0 && env.client_blocked(i, cur_iters[i])) {
                seen[i] = num_kernels[i];
                stats.forced_iter_ends++;
                continue;
            }
            int t = env.peek(i);
            if (t >= 0) {
                heads[i] = t;
                int cur = cur_iters[i];
                if (seen[i] == 0 && !starts_set[i][cur]) {
                    client_starts[i] = env.now_us();
                    starts_set[i][cur] = 1;
                    if (!total_client_set[i]) {
                        total_client_starts[i] = env.now_us();
                        total_client_set[i] = 1;
                    }
                }
            }
        }

        if (reef) {
            schedule_reef(env, heads, depth);
        } else if (seq) {
            start = schedule_sequential(env, heads, start);
        } else {
            if (heads[hp] >= 0) {
                const OpInfo& op1 = op_info[hp][seen[hp]];
                int prof = op1.profile;
                hp_sm_need = op1.sm_used;
                submit(env, heads[hp], hp, hp, hp);
                profiles[hp] = prof;
                stats.hp_submits++;
            }
            int end = start + n;
            for (int t = start + 1; t < end; t++) {
                int j = t % (n - 1);   // never reached with one client: the range is empty
                if (heads[j] < 0) continue;
                const OpInfo& op0 = op_info[j][seen[j]];
                const int type = heads[j];
                const bool memop = orion_is_memop(type);
                bool go = false;
                if (seen[hp] == 0 || memop)
                    go = true;
                else if (cur_iters[j] <= 10 || cur_iters[hp] >= max_iters[hp])
                    go = true;
                else if (seen[hp] >= update_start && op0.sm_used <= sm_threshold &&
                         (stats.queries++, env.query(hp, update_start - 1)))
                    go = true;
                else if (seen[hp] > 0 && (size + op0.sm_used <= sm_threshold) &&
                         (op0.profile == -1 || profiles[hp] == -1 || profiles[hp] != op0.profile))
                    go = true;
                if (go && large_found) {
                    bool drained = true;
                    for (int k = 0; k < n - 1; k++) {
                        if (event_ids[k] >= 1) {
                            stats.queries++;
                            if (!env.query(k, event_ids[k] - 1)) {
                                drained = false;
                                break;
                            }
                        }
                    }
                    if (drained) {
                        large_found = false;
                        sum = 0;
                    } else {
                        go = false;
                    }
                }
                if (go) {
                    size += op0.sm_used;
                    if (!memop) sum = (long)((float)sum + op0.duration);
                    if (sum > depth && cur_iters[hp] < max_iters[hp]) large_found = true;
                    submit(env, type, j, j, j);
                    stats.be_submits++;
                    start = j;
                } else {
                    stats.be_rejects++;
                }
            }
        }
        if (error) return;

        int finished = 0;
        for (int i = 0; i < n; i++) {
            if (cur_iters[i] == max_iters[i] || (warmup && cur_iters[i] == a.warmup_iters) || env.stop_ack(i)) {
                finished += 1;
            } else if (seen[i] == num_kernels[i]) {
                if (!locked[i]) {
                    env.iter_lock(i);
                    locked[i] = 1;
                }
                bool ready = true;
                int evl = seq ? 0 : i;
                if (event_ids[evl] >= 1) {
                    stats.queries++;
                    if (!env.query(evl, event_ids[evl] - 1)) ready = false;
                }
                if (ready) {
                    closed_iter = true;
                    seen[i] = 0;
                    if (seq) event_ids[0] = 0;
                    event_ids[i] = 0;
                    env.iter_done(i, cur_iters[i]);
                    cur_iters[i] += 1;
                    locked[i] = 0;

                    float duration = (float)(env.now_us() - client_starts[i]);
                    duration /= 1000.0;
                    client_durations[i].push_back(duration);
                    if (!reef && !seq && i == hp && is_train[hp]) {
                        // Bisection of the SM threshold against the tolerated HP
                        // iteration time, every 10 HP training iterations.
                        hp_iter_duration += duration;
                        if ((cur_iters[i] % 10) == 0 && low_sms != sm_threshold) {
                            float hp_avg = hp_iter_duration / 10.0;
                            hp_iter_duration = 0;
                            if (hp_avg > hp_limit_float) {
                                high_sms = sm_threshold;
                                sm_threshold = (low_sms + high_sms) / 2;
                            } else {
                                low_sms = sm_threshold;
                                sm_threshold = (low_sms + high_sms) / 2;
                            }
                        }
                    }
                }
                if (cur_iters[i] == max_iters[i] || (warmup && cur_iters[i] == a.warmup_iters) ||
                    env.stop_ack(i)) {
                    finished += 1;
                    if (!warmup && i == n - 1) {
                        for (int k = 0; k < n - 1; k++) env.stop(k, locked[k] != 0);
                    }
                }
            }
        }
        if (finished == n) break;
        env.poll_end(closed_iter || released != released_before);
    }
}

}  // namespace orion
