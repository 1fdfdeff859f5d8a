// Loader for the per-kernel profile files of benchmarking/model_kernels
// (header `Name,Profile,Memory_footprint,SM_usage,Duration`, one row per
// scheduled compute op in launch order).
//
// Behaviour follows populate_kernel_info (src/scheduler/scheduler_eval.cpp:498-526):
// the first line is dropped unseen, every other line is split on ',' and fields
// 1..3 go through stoi and field 4 through stof, so "12abc" parses as 12 and a
// non-numeric field throws.  Where the reference indexes past the end of a short
// row (undefined behaviour) this loader reports the line instead.
#pragma once
#include <fstream>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace orion {

struct OpInfo {            // src/scheduler/utils_sched.h:90-98
    std::string name;
    int profile;           // 1 compute-bound, 0 memory-bound, -1 unclear
    int mem;
    int sm_used;
    float duration;        // ns, stored as float exactly as the reference does
};

inline std::vector<std::string> split_commas(const std::string& line) {
    // Same loop shape as the reference: getline on ',' while the stream is good,
    // which yields one (possibly empty) trailing field for "a,b,".
    std::vector<std::string> v;
    std::stringstream s(line);
    while (s.good()) {
        std::string f;
        std::getline(s, f, ',');
        v.push_back(f);
    }
    return v;
}

inline void load_profile(const std::string& path, std::vector<OpInfo>& ops) {
    std::ifstream in(path);
    if (!in.is_open()) throw std::runtime_error("orion: cannot open profile file " + path);
    std::string line;
    std::getline(in, line);  // header
    size_t lineno = 1;
    while (std::getline(in, line)) {
        ++lineno;
        std::vector<std::string> v = split_commas(line);
        if (v.size() < 5)
            throw std::runtime_error("orion: profile " + path + " line " + std::to_string(lineno) +
                                     ": expected 5 comma-separated fields");
        OpInfo o{v[0], std::stoi(v[1]), std::stoi(v[2]), std::stoi(v[3]), std::stof(v[4])};
        ops.push_back(std::move(o));
    }
}

inline int max_sm_used(const std::vector<OpInfo>& ops) {
    int m = 0;
    for (const OpInfo& o : ops) m = o.sm_used > m ? o.sm_used : m;
    return m;
}

}  // namespace orion
