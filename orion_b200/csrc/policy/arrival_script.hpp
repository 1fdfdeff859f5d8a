// Closed-loop arrival scripts: the input of the virtual-time simulator that
// drives a scheduling policy without a GPU or client threads.
//
// A script names, per client, the op sequence of one request/iteration (record
// type, host gap before the push, simulated device duration), the profile file
// the scheduler is given for it, and how requests arrive.  Time is counted in
// ticks; one tick is one microsecond of the simulated clock.
//
// Text format (whitespace separated; '#' starts a comment to end of line):
//   orion_script 1
//   algo orion|reef|sequential
//   depth <int>  hp_limit <int>  update_start <int>  max_sms <int>
//   nclients <N>
//   client <i>
//     train <0|1>  num_iters <M>  think <ticks>
//     profile <path> <num_kernels>
//     [profile2 <path> <num_kernels>]      installed after the first phase
//     [ops0 <n> (<type> <gap> <dur>)*n]    op sequence of iteration 0
//     ops <n> (<type> <gap> <dur>)*n       op sequence of every later iteration
//     gaps closed | gaps open <M ints>     minimum distance between request starts
//   end
//   phases <P> (<warmup 0|1> <warmup_iters>)*P
// Paths are relative to the directory of the script file.
#pragma once
#include <cstdint>
#include <fstream>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace orion {

struct ScriptOp {
    int type;
    int64_t gap;   // ticks between "previous op popped" and "this op visible in the queue"
    int64_t dur;   // simulated device time in ticks
};

struct ScriptClient {
    bool train = false;
    int num_iters = 0;
    int64_t think = 0;
    std::string profile, profile2;
    int num_kernels = 0, num_kernels2 = -1;
    std::vector<ScriptOp> ops0, ops;
    std::vector<int64_t> gaps;   // empty = closed loop
};

struct ScriptPhase {
    bool warmup;
    int warmup_iters;
};

struct ArrivalScript {
    std::string algo = "orion";
    int depth = 1, hp_limit = 1, update_start = 1, max_sms = 80;
    std::vector<ScriptClient> clients;
    std::vector<ScriptPhase> phases;
    std::string dir;
};

inline ArrivalScript load_script(const std::string& path) {
    std::ifstream in(path);
    if (!in.is_open()) throw std::runtime_error("orion: cannot open script " + path);
    std::stringstream toks;
    std::string line;
    while (std::getline(in, line)) {
        size_t h = line.find('#');
        if (h != std::string::npos) line.resize(h);
        toks << line << '\n';
    }
    ArrivalScript s;
    size_t slash = path.find_last_of('/');
    s.dir = slash == std::string::npos ? "." : path.substr(0, slash);
    auto need = [&](auto& v, const char* what) {
        if (!(toks >> v)) throw std::runtime_error(std::string("orion: script ") + path + ": expected " + what);
    };
    auto rel = [&](const std::string& p) { return (!p.empty() && p[0] == '/') ? p : s.dir + "/" + p; };
    auto read_ops = [&](std::vector<ScriptOp>& ops) {
        int n;
        need(n, "op count");
        ops.resize(n);
        for (ScriptOp& o : ops) {
            need(o.type, "op type");
            need(o.gap, "op gap");
            need(o.dur, "op dur");
        }
    };
    std::string key;
    int version = 0;
    need(key, "orion_script");
    need(version, "version");
    if (key != "orion_script" || version != 1) throw std::runtime_error("orion: not an arrival script: " + path);
    while (toks >> key) {
        if (key == "algo") need(s.algo, "algo");
        else if (key == "depth") need(s.depth, "depth");
        else if (key == "hp_limit") need(s.hp_limit, "hp_limit");
        else if (key == "update_start") need(s.update_start, "update_start");
        else if (key == "max_sms") need(s.max_sms, "max_sms");
        else if (key == "nclients") {
            int n;
            need(n, "nclients");
            s.clients.resize(n);
        } else if (key == "client") {
            int i;
            need(i, "client index");
            if (i < 0 || i >= (int)s.clients.size()) throw std::runtime_error("orion: script client index out of range");
            ScriptClient& c = s.clients[i];
            while (true) {
                need(key, "client field");
                if (key == "end") break;
                else if (key == "train") { int t; need(t, "train"); c.train = t != 0; }
                else if (key == "num_iters") need(c.num_iters, "num_iters");
                else if (key == "think") need(c.think, "think");
                else if (key == "profile") { need(c.profile, "profile"); c.profile = rel(c.profile); need(c.num_kernels, "num_kernels"); }
                else if (key == "profile2") { need(c.profile2, "profile2"); c.profile2 = rel(c.profile2); need(c.num_kernels2, "num_kernels2"); }
                else if (key == "ops0") read_ops(c.ops0);
                else if (key == "ops") read_ops(c.ops);
                else if (key == "gaps") {
                    std::string mode;
                    need(mode, "gaps mode");
                    if (mode == "open") {
                        c.gaps.resize(c.num_iters);
                        for (int64_t& g : c.gaps) need(g, "gap");
                    } else if (mode != "closed") throw std::runtime_error("orion: script gaps must be open|closed");
                } else throw std::runtime_error("orion: unknown client field " + key);
            }
        } else if (key == "phases") {
            int p;
            need(p, "phase count");
            s.phases.resize(p);
            for (ScriptPhase& ph : s.phases) {
                int w;
                need(w, "warmup flag");
                need(ph.warmup_iters, "warmup_iters");
                ph.warmup = w != 0;
            }
        } else throw std::runtime_error("orion: unknown script key " + key);
    }
    if (s.clients.empty() || s.phases.empty()) throw std::runtime_error("orion: script needs clients and phases");
    return s;
}

}  // namespace orion
