// Virtual-time environment for PolicyCore: simulated clients that obey the
// depth-1 closed loop of the capture shim (a client pushes its next op only
// after the previous one was popped), one FIFO device timeline per stream, and
// events that complete when the work submitted before them has drained.
//
// Clock rule: the clock advances by one tick on every queue-lock the scheduler
// takes outside a pop (peek, end-of-iteration lock, stop), on every submit and
// on every event query.  A scheduler that issues a different sequence of such
// calls therefore sees different times — which makes the decision log of a run
// a fingerprint of the whole call sequence, not only of the admitted ops.
//
// Log lines (one per event, in order):
//   S <tick> <client> <type> <stream> <ev_list> <ev_slot>    op released
//   Q <tick> <ev_list> <ev_slot> <0|1>                       event query and answer
//   D <tick> <client> <iter>                                 request/iteration complete
//   X <tick> <client>                                        stop requested
//   E <phase>                                                schedule() returned
#pragma once
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

#include "arrival_script.hpp"
#include "op_types.h"

namespace orion {

struct LogRec {
    char kind;
    int64_t a, b, c, d, e, f;
};

class DecisionLog {
public:
    std::vector<LogRec> recs;
    void add(char k, int64_t a = 0, int64_t b = 0, int64_t c = 0, int64_t d = 0, int64_t e = 0, int64_t f = 0) {
        recs.push_back(LogRec{k, a, b, c, d, e, f});
    }
    static int format(const LogRec& r, char* buf, size_t n) {
        switch (r.kind) {
            case 'S': return snprintf(buf, n, "S %ld %ld %ld %ld %ld %ld\n", (long)r.a, (long)r.b, (long)r.c, (long)r.d, (long)r.e, (long)r.f);
            case 'Q': return snprintf(buf, n, "Q %ld %ld %ld %ld\n", (long)r.a, (long)r.b, (long)r.c, (long)r.d);
            case 'D': return snprintf(buf, n, "D %ld %ld %ld\n", (long)r.a, (long)r.b, (long)r.c);
            case 'X': return snprintf(buf, n, "X %ld %ld\n", (long)r.a, (long)r.b);
            default: return snprintf(buf, n, "E %ld\n", (long)r.a);
        }
    }
    uint64_t fnv1a() const {
        uint64_t h = 1469598103934665603ull;
        char buf[160];
        for (const LogRec& r : recs) {
            int len = format(r, buf, sizeof buf);
            for (int i = 0; i < len; i++) {
                h ^= (unsigned char)buf[i];
                h *= 1099511628211ull;
            }
        }
        return h;
    }
    bool write(const std::string& path) const {
        FILE* f = fopen(path.c_str(), "w");
        if (!f) return false;
        char buf[160];
        for (const LogRec& r : recs) {
            int len = format(r, buf, sizeof buf);
            fwrite(buf, 1, (size_t)len, f);
        }
        fclose(f);
        return true;
    }
    size_t count(char k) const {
        size_t c = 0;
        for (const LogRec& r : recs) c += r.kind == k;
        return c;
    }
};

class SimEnv {
public:
    static constexpr int kEventsPerList = 30000;   // utils_sched.cpp:150

    struct Client {
        const ScriptClient* sc = nullptr;
        int it = 0;            // iteration being issued
        int k = 0;             // next op of that iteration
        bool in_queue = false;
        bool waiting_done = false;
        bool stopped = false;
        bool stop_flag = false;
        bool stop_ack = false;
        int64_t next_push_at = 0;
        int64_t iter_earliest = 0;
        int iter_limit = 0;
        std::vector<char> request_status;   // what block(it) spins on in the real client
    };

    int64_t now = 0;
    std::vector<Client> clients;
    std::vector<int64_t> busy;                      // per stream
    std::vector<std::vector<int64_t>> done_at;      // per event list / slot
    DecisionLog log;
    bool broken = false;                            // the policy asked for something impossible

    explicit SimEnv(const ArrivalScript& s) {
        int n = (int)s.clients.size();
        clients.resize(n);
        busy.assign(n, 0);
        done_at.assign(n, std::vector<int64_t>(kEventsPerList, 0));
        for (int i = 0; i < n; i++) {
            clients[i].sc = &s.clients[i];
            clients[i].request_status.assign((size_t)s.clients[i].num_iters + 1, 0);
            clients[i].next_push_at = seq_of(clients[i]).empty() ? 0 : seq_of(clients[i])[0].gap;
        }
    }

    void begin_phase(const ScriptPhase& p) {
        for (Client& c : clients) c.iter_limit = p.warmup ? p.warmup_iters : c.sc->num_iters;
    }
    void end_phase(int phase) { log.add('E', phase); }

    // ---- Env interface ----
    int peek(int i) {
        touch(i);
        Client& c = clients[i];
        int head = c.in_queue ? seq_of(c)[c.k].type : -1;
        after_unlock(i);
        return head;
    }
    int64_t now_us() const { return now; }
    void submit(int i, int type, int stream, int evl, int evs) {
        now += 1;
        Client& c = clients[i];
        const std::vector<ScriptOp>& ops = seq_of(c);
        if (!c.in_queue || ops[c.k].type != type) {
            broken = true;
            return;
        }
        const ScriptOp& op = ops[c.k];
        int64_t start = std::max(now, busy[stream]);
        busy[stream] = start + op.dur;
        done_at[evl][evs] = busy[stream];
        log.add('S', now, i, type, stream, evl, evs);
        c.in_queue = false;
        c.k += 1;
        if (c.k == (int)ops.size())
            c.waiting_done = true;
        else
            c.next_push_at = now + ops[c.k].gap;
        after_unlock(i);
    }
    bool query(int evl, int evs) {
        now += 1;
        bool done = now >= done_at[evl][evs];
        log.add('Q', now, evl, evs, done ? 1 : 0);
        return done;
    }
    void iter_lock(int i) { touch(i); }
    void iter_done(int i, int iter) {
        clients[i].request_status[(size_t)iter] = 1;
        after_unlock(i);
    }
    void stop(int k, bool locked) {
        if (!locked) touch(k);
        clients[k].stop_flag = true;
        log.add('X', now, k);
        if (!locked) after_unlock(k);
    }
    bool stop_ack(int i) const { return clients[i].stop_ack; }
    bool client_blocked(int, int) const { return false; }
    void poll_end(bool) {}

private:
    const std::vector<ScriptOp>& seq_of(const Client& c) const {
        return (c.it == 0 && !c.sc->ops0.empty()) ? c.sc->ops0 : c.sc->ops;
    }
    // A simulated client notices a finished request the next time its queue lock is
    // released after (a) all its ops were popped and (b) the scheduler flagged the
    // request.  (b) can precede (a) when an iteration ends in memory ops, which the
    // scheduler does not count.
    void after_unlock(int i) {
        Client& c = clients[i];
        if (!c.waiting_done || !c.request_status[(size_t)c.it]) return;
        log.add('D', now, i, c.it);
        int64_t prev_start = c.iter_earliest;
        int64_t gap = c.sc->gaps.empty() ? 0 : c.sc->gaps[(size_t)c.it];
        c.it += 1;
        c.k = 0;
        c.waiting_done = false;
        if (c.stop_flag) {
            c.stop_ack = true;
            c.stopped = true;
            return;
        }
        c.iter_earliest = std::max(now + c.sc->think, prev_start + gap);
        const std::vector<ScriptOp>& ops = seq_of(c);
        c.next_push_at = c.iter_earliest + (ops.empty() ? 0 : ops[0].gap);
    }
    void touch(int i) {
        now += 1;
        Client& c = clients[i];
        if (!c.in_queue && !c.waiting_done && !c.stopped && c.it < c.iter_limit && c.it < c.sc->num_iters &&
            now >= c.next_push_at && !seq_of(c).empty())
            c.in_queue = true;
    }
};

}  // namespace orion
