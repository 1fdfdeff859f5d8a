// Observation traces: what the live scheduler saw and what it decided, poll by poll.
//
// The policy (policy.hpp) touches the outside world through an Env.  `ObsEnv` wraps the live Env, forwards every
// call and writes down, in call order,
//   inputs   P<i>:<type>          answer of peek(i) (-1 = empty queue); types as the reference numbers them
//            Q<list>:<slot>:<0|1> answer of an event query
//            T<microseconds>      a clock read
//            K<mask>              stop acknowledgements in force from this poll on (bit i = client i)
//            B<i>                 client_blocked(i) was true: the iteration was closed early (the reference cannot
//                                 do that; a trace with a B token is not comparable past it)
//   outputs  S<i>:<type>:<stream>:<list>:<slot>   an op released
//            L<i>                 the iteration-end lock taken
//            D<i>:<iter>          a request / iteration closed
//            X<k>:<locked>        client k asked to stop
// One text line per poll, `p <repeat> <tokens...>`; consecutive polls that saw the same answers and released
// nothing are folded into one line with a repeat count.  `phase`, `reset` and `setup_change` lines carry the calls
// between polls.  The checker oracle/ref_driver.cpp feeds the inputs to the compiled reference scheduler
// (src/scheduler/scheduler_eval.cpp) at the very calls where it would have asked for them and compares the outputs,
// so the decisions taken live are compared, not a re-simulation of them.
//
// Stop acknowledgements are sampled once per poll while a trace is recorded: the reference reads its flag from
// memory, which the checker can only change between two of the reference's calls.
#pragma once
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <stdlib.h>

#include <fstream>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "../policy/op_types.h"

namespace orion {

struct ObsToken {
    int32_t kind, a, b, c, d, e;
    int64_t t;
    bool operator==(const ObsToken& o) const {
        return kind == o.kind && a == o.a && b == o.b && c == o.c && d == o.d && e == o.e && t == o.t;
    }
};

class ObsRecorder {
public:
    FILE* f = nullptr;
    uint64_t max_lines = 0, lines = 0, polls = 0;
    bool truncated = false;

    bool open(const char* path, uint64_t cap) {
        f = fopen(path, "w");
        max_lines = cap;
        return f != nullptr;
    }
    bool on() const { return f != nullptr && !truncated; }
    void raw(const std::string& line) {
        if (!f) return;
        flush_prev();
        fputs(line.c_str(), f);
        fputc('\n', f);
    }
    void add(char kind, int a = 0, int b = 0, int c = 0, int d = 0, int e = 0, int64_t t = 0) {
        if (!on()) return;
        cur.push_back(ObsToken{kind, a, b, c, d, e, t});
        if (kind != 'P' && kind != 'Q') cur_pure = false;
    }
    void end_poll() {
        if (!on()) return;
        polls++;
        if (cur_pure && prev_pure && prev_rep > 0 && cur == prev) {
            prev_rep++;
        } else {
            flush_prev();
            prev.swap(cur);
            prev_pure = cur_pure;
            prev_rep = 1;
        }
        cur.clear();
        cur_pure = true;
    }
    void close() {
        if (!f) return;
        flush_prev();
        if (truncated) fputs("truncated\n", f);
        fclose(f);
        f = nullptr;
    }

private:
    std::vector<ObsToken> cur, prev;
    uint64_t prev_rep = 0;
    bool cur_pure = true, prev_pure = false;

    void flush_prev() {
        if (prev_rep == 0) return;
        fprintf(f, "p %llu", (unsigned long long)prev_rep);
        for (const ObsToken& k : prev) {
            switch (k.kind) {
                case 'P': fprintf(f, " P%d:%d", k.a, k.b); break;
                case 'Q': fprintf(f, " Q%d:%d:%d", k.a, k.b, k.c); break;
                case 'T': fprintf(f, " T%lld", (long long)k.t); break;
                case 'K': fprintf(f, " K%d", k.a); break;
                case 'B': fprintf(f, " B%d", k.a); break;
                case 'S': fprintf(f, " S%d:%d:%d:%d:%d", k.a, k.b, k.c, k.d, k.e); break;
                case 'L': fprintf(f, " L%d", k.a); break;
                case 'D': fprintf(f, " D%d:%d", k.a, k.b); break;
                case 'X': fprintf(f, " X%d:%d", k.a, k.b); break;
            }
        }
        fputc('\n', f);
        prev_rep = 0;
        prev.clear();
        if (max_lines && ++lines >= max_lines) truncated = true;
    }
};

template <class Inner>
struct ObsEnv {
    Inner& in;
    ObsRecorder& rec;
    int n;
    uint32_t ack_mask = 0;
    bool mask_known = false;

    ObsEnv(Inner& inner, ObsRecorder& r, int clients) : in(inner), rec(r), n(clients) {}

    void sample_acks() {
        uint32_t m = 0;
        for (int i = 0; i < n; i++)
            if (in.stop_ack(i)) m |= 1u << i;
        if (!mask_known || m != ack_mask) rec.add('K', (int)m);
        ack_mask = m;
        mask_known = true;
    }
    void begin_phase() { sample_acks(); }
    void end_phase() { rec.end_poll(); }

    int peek(int i) {
        int t = in.peek(i);
        rec.add('P', i, t < 0 ? -1 : orion_reference_type(t));
        return t;
    }
    int64_t now_us() {
        int64_t t = in.now_us();
        rec.add('T', 0, 0, 0, 0, 0, t);
        return t;
    }
    void submit(int i, int type, int stream, int evl, int evs) {
        rec.add('S', i, orion_reference_type(type), stream, evl, evs);
        in.submit(i, type, stream, evl, evs);
    }
    bool query(int evl, int evs) {
        bool r = in.query(evl, evs);
        rec.add('Q', evl, evs, r ? 1 : 0);
        return r;
    }
    void iter_lock(int i) {
        rec.add('L', i);
        in.iter_lock(i);
    }
    void iter_done(int i, int iter) {
        rec.add('D', i, iter);
        in.iter_done(i, iter);
    }
    void stop(int k, bool locked) {
        rec.add('X', k, locked ? 1 : 0);
        in.stop(k, locked);
    }
    bool stop_ack(int i) { return (ack_mask >> i) & 1u; }
    bool client_blocked(int i, int iter) {
        bool b = in.client_blocked(i, iter);
        if (b) rec.add('B', i);
        return b;
    }
    void poll_end(bool progressed) {
        rec.end_poll();
        sample_acks();
        in.poll_end(progressed);
    }
};

// ---------------------------------------------------------------------------------------------------------------------
// Reading a trace back, and an Env that replays it: the policy core gets the recorded answers and every call it makes
// (release, lock, closed request, stop) is compared with the recorded one.  Used by `orion_replay --observations`.

struct ObsTraceLine {
    uint64_t rep = 1;
    std::vector<ObsToken> toks;
};
struct ObsTraceCmd {
    bool is_phase = true;            // else: setup_change
    int args[7] = {0, 0, 0, 0, 0, 0, 0};   // phase: warmup, warmup_iters, reef, seq, depth, hp_limit, update_start
    std::vector<ObsTraceLine> lines;
    int client = 0, num_kernels = 0;
    std::string file;
};
struct ObsTrace {
    int max_sms = 80, reef = 0, n = 0;
    std::vector<int> num_kernels, num_iters, train;
    std::vector<std::string> profiles;
    std::vector<ObsTraceCmd> cmds;
    bool truncated = false;
};

// Throws std::runtime_error on a malformed file.  Profile paths that are not absolute are taken relative to the trace.
inline ObsTrace load_obs_trace(const std::string& path) {
    std::ifstream in(path);
    if (!in.is_open()) throw std::runtime_error("orion: cannot open observation trace " + path);
    const size_t slash = path.find_last_of('/');
    const std::string dir = slash == std::string::npos ? "." : path.substr(0, slash);
    auto rel = [&](const std::string& p) { return (!p.empty() && p[0] == '/') ? p : dir + "/" + p; };
    ObsTrace t;
    std::string line, key, k;
    while (std::getline(in, line)) {
        std::istringstream ls(line);
        if (!(ls >> key)) continue;
        if (key == "orion_observations" || key == "endphase" || key == "reset") continue;
        if (key == "max_sms") {
            ls >> t.max_sms >> k >> t.reef;
        } else if (key == "nclients") {
            ls >> t.n;
            t.num_kernels.assign(t.n, 0);
            t.num_iters.assign(t.n, 0);
            t.train.assign(t.n, 0);
            t.profiles.assign(t.n, "");
        } else if (key == "client") {
            int i = -1;
            ls >> i;
            if (i < 0 || i >= t.n) throw std::runtime_error("orion: observation trace names a client out of range");
            ls >> k >> t.train[i] >> k >> t.num_iters[i] >> k >> t.profiles[i] >> t.num_kernels[i];
            t.profiles[i] = rel(t.profiles[i]);
        } else if (key == "phase") {
            ObsTraceCmd c;
            for (int a = 0; a < 7; a++) ls >> c.args[a];
            t.cmds.push_back(c);
        } else if (key == "setup_change") {
            ObsTraceCmd c;
            c.is_phase = false;
            ls >> c.client >> c.file >> c.num_kernels;
            c.file = rel(c.file);
            t.cmds.push_back(c);
        } else if (key == "truncated") {
            t.truncated = true;
        } else if (key == "p") {
            if (t.cmds.empty() || !t.cmds.back().is_phase) throw std::runtime_error("orion: poll line outside a phase");
            ObsTraceLine l;
            ls >> l.rep;
            std::string w;
            while (ls >> w) {
                ObsToken tk{w[0], 0, 0, 0, 0, 0, 0};
                const char* p = w.c_str() + 1;
                if (tk.kind == 'T') {
                    tk.t = strtoll(p, nullptr, 10);
                } else {
                    int32_t* f[5] = {&tk.a, &tk.b, &tk.c, &tk.d, &tk.e};
                    for (int q = 0; q < 5 && *p; q++) {
                        char* end = nullptr;
                        *f[q] = (int32_t)strtol(p, &end, 10);
                        p = (*end == ':') ? end + 1 : end;
                    }
                }
                if (!strchr("PQTKBSLDX", tk.kind)) throw std::runtime_error("orion: unknown token in observation trace");
                l.toks.push_back(tk);
            }
            if (!l.toks.empty() && l.rep > 0) t.cmds.back().lines.push_back(l);
        } else {
            throw std::runtime_error("orion: unknown line in observation trace: " + key);
        }
    }
    if (t.n < 1 || t.cmds.empty()) throw std::runtime_error("orion: observation trace holds no phase");
    return t;
}

struct ObsMismatch {
    bool exhausted;        // the trace ended (recording limit) before the policy did
    std::string detail;
};

struct ObsReplayEnv {
    const std::vector<ObsTraceLine>* lines = nullptr;
    size_t line = 0, tok = 0;
    uint64_t rep = 0;
    uint32_t ack = 0;
    int64_t last_t = 0;
    uint64_t decisions = 0, closed = 0, polls = 0;

    void begin(const std::vector<ObsTraceLine>* l) {
        lines = l;
        line = tok = 0;
        rep = 0;
    }
    const ObsToken* cur() {
        while (line < lines->size()) {
            const ObsTraceLine& l = (*lines)[line];
            if (tok < l.toks.size()) {
                if (l.toks[tok].kind == 'K') {   // stop acknowledgements in force from this poll on
                    ack = (uint32_t)l.toks[tok].a;
                    tok++;
                    continue;
                }
                return &l.toks[tok];
            }
            tok = 0;
            polls++;
            if (++rep >= l.rep) {
                rep = 0;
                line++;
            }
        }
        return nullptr;
    }
    const ObsToken& expect(char kind, int a, const char* what) {
        const ObsToken* t = cur();
        if (!t) throw ObsMismatch{true, std::string("the trace ends before a ") + what};
        if (t->kind != kind || t->a != a)
            throw ObsMismatch{false, std::string(what) + ": the policy core asks for " + kind + std::to_string(a) + ", the trace holds " +
                                         (char)t->kind + std::to_string(t->a)};
        tok++;
        return *t;
    }
    bool drained() { return cur() == nullptr; }

    int peek(int i) { return expect('P', i, "queue head").b; }
    int64_t now_us() {
        const ObsToken* t = cur();
        if (t && t->kind == 'T') {
            last_t = t->t;
            tok++;
        }
        return last_t;
    }
    void submit(int i, int type, int stream, int evl, int evs) {
        const ObsToken& t = expect('S', i, "release");
        if (t.b != orion_reference_type(type) || t.c != stream || t.d != evl || t.e != evs)
            throw ObsMismatch{false, "release of client " + std::to_string(i) + " differs in type, stream or event"};
        decisions++;
    }
    bool query(int evl, int evs) {
        const ObsToken& t = expect('Q', evl, "event query");
        if (t.b != evs) throw ObsMismatch{false, "event query of another slot"};
        return t.c != 0;
    }
    void iter_lock(int i) { expect('L', i, "iteration lock"); }
    void iter_done(int i, int iter) {
        if (expect('D', i, "closed request").b != iter) throw ObsMismatch{false, "closed request of another index"};
        closed++;
    }
    void stop(int k, bool locked) {
        if (expect('X', k, "stop request").b != (locked ? 1 : 0)) throw ObsMismatch{false, "stop request with another lock state"};
    }
    bool stop_ack(int i) { return (ack >> i) & 1u; }
    bool client_blocked(int i, int) {
        const ObsToken* t = cur();
        if (t && t->kind == 'B' && t->a == i) {
            tok++;
            return true;
        }
        return false;
    }
    void poll_end(bool) {}
};

}  // namespace orion
