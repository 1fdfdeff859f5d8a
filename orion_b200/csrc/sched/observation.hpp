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

}  // namespace orion
