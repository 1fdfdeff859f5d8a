"""TEST INFRASTRUCTURE — a CPU restatement of the reference scheduling policy.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline leg may import
this file; the product never does.

`run_script(path)` replays an arrival script (format: see
orion_b200/csrc/policy/arrival_script.hpp) through a pure-Python restatement of
  * Scheduler::busy_wait_profile   src/scheduler/scheduler_eval.cpp:238-487
  * Scheduler::schedule_reef       src/scheduler/scheduler_eval.cpp:93-165
  * Scheduler::schedule_sequential src/scheduler/scheduler_eval.cpp:167-236
  * schedule_kernel's counters     src/scheduler/utils_sched.cpp:239-522
  * populate_kernel_info           src/scheduler/scheduler_eval.cpp:498-526
and returns the decision log as text.  The virtual-time client/device model is
the one documented in oracle/ref_driver.cpp: one tick per non-pop queue lock,
per submit and per event query.

Pinned: tests/test_policy_parity.py checks this restatement against the logs in
tests/golden/, which were produced by the reference's own scheduler sources
compiled unmodified (oracle/Makefile, oracle/ref_driver.cpp).
"""
import hashlib
import os

import numpy as np

INT_MAX = 2**31 - 1
MEMOPS = (1, 2, 3, 4)          # MEMCPY, MALLOC, FREE, MEMSET (intercept_temp.h:642-660)
MALLOC = 2
UNSUPPORTED = (5, 8)           # utils_sched.cpp:514-516 aborts on these
EVENTS_PER_LIST = 30000        # utils_sched.cpp:150
f32 = np.float32


def stoi(s):
    """std::stoi: optional whitespace, sign, then as many digits as there are."""
    s = s.lstrip()
    i = 1 if s[:1] in "+-" else 0
    j = i
    while j < len(s) and s[j].isdigit():
        j += 1
    if j == i:
        raise ValueError("stoi: no conversion: %r" % s)
    return int(s[:j])


def load_profile(path):
    """populate_kernel_info (scheduler_eval.cpp:498-526)."""
    ops = []
    with open(path) as f:
        f.readline()
        for line in f:
            v = line.rstrip("\n").split(",")
            ops.append((v[0], stoi(v[1]), stoi(v[2]), stoi(v[3]), f32(float(v[4]))))
    return ops


def parse_script(path):
    toks = []
    with open(path) as f:
        for line in f:
            toks += line.split("#", 1)[0].split()
    d = os.path.dirname(os.path.abspath(path))
    pos = [0]

    def nxt():
        pos[0] += 1
        return toks[pos[0] - 1]

    assert nxt() == "orion_script" and nxt() == "1"
    s = dict(algo="orion", depth=1, hp_limit=1, update_start=1, max_sms=80, clients=[], phases=[])

    def read_ops():
        n = int(nxt())
        return [(int(nxt()), int(nxt()), int(nxt())) for _ in range(n)]

    while pos[0] < len(toks):
        k = nxt()
        if k == "algo":
            s["algo"] = nxt()
        elif k in ("depth", "hp_limit", "update_start", "max_sms"):
            s[k] = int(nxt())
        elif k == "nclients":
            s["clients"] = [dict(train=False, num_iters=0, think=0, profile2=None, ops0=[], ops=[], gaps=[])
                            for _ in range(int(nxt()))]
        elif k == "client":
            c = s["clients"][int(nxt())]
            while True:
                k = nxt()
                if k == "end":
                    break
                if k == "train":
                    c["train"] = nxt() != "0"
                elif k in ("num_iters", "think"):
                    c[k] = int(nxt())
                elif k == "profile":
                    c["profile"] = os.path.join(d, nxt())
                    c["num_kernels"] = int(nxt())
                elif k == "profile2":
                    c["profile2"] = os.path.join(d, nxt())
                    c["num_kernels2"] = int(nxt())
                elif k == "ops0":
                    c["ops0"] = read_ops()
                elif k == "ops":
                    c["ops"] = read_ops()
                elif k == "gaps":
                    if nxt() == "open":
                        c["gaps"] = [int(nxt()) for _ in range(c["num_iters"])]
                else:
                    raise ValueError(k)
        elif k == "phases":
            s["phases"] = [(nxt() != "0", int(nxt())) for _ in range(int(nxt()))]
        else:
            raise ValueError(k)
    return s


class Sim:
    """Virtual-time clients and device (rules in oracle/ref_driver.cpp)."""

    def __init__(self, script):
        n = len(script["clients"])
        self.now = 0
        self.log = []
        self.c = []
        for sc in script["clients"]:
            c = dict(sc=sc, it=0, k=0, in_queue=False, waiting=False, stopped=False, stop_flag=False,
                     stop_ack=False, earliest=0, limit=0, status=[False] * (sc["num_iters"] + 1))
            seq = self._seq(c)
            c["next_push"] = seq[0][1] if seq else 0
            self.c.append(c)
        self.busy = [0] * n
        self.done_at = {}

    @staticmethod
    def _seq(c):
        return c["sc"]["ops0"] if (c["it"] == 0 and c["sc"]["ops0"]) else c["sc"]["ops"]

    def _touch(self, i):
        self.now += 1
        c = self.c[i]
        if (not c["in_queue"] and not c["waiting"] and not c["stopped"] and c["it"] < c["limit"]
                and c["it"] < c["sc"]["num_iters"] and self.now >= c["next_push"] and self._seq(c)):
            c["in_queue"] = True

    def _after_unlock(self, i):
        c = self.c[i]
        if not c["waiting"] or not c["status"][c["it"]]:
            return
        self.log.append("D %d %d %d" % (self.now, i, c["it"]))
        prev = c["earliest"]
        gap = c["sc"]["gaps"][c["it"]] if c["sc"]["gaps"] else 0
        c["it"] += 1
        c["k"] = 0
        c["waiting"] = False
        if c["stop_flag"]:
            c["stop_ack"] = c["stopped"] = True
            return
        c["earliest"] = max(self.now + c["sc"]["think"], prev + gap)
        seq = self._seq(c)
        c["next_push"] = c["earliest"] + (seq[0][1] if seq else 0)

    def peek(self, i):
        self._touch(i)
        c = self.c[i]
        head = self._seq(c)[c["k"]][0] if c["in_queue"] else -1
        self._after_unlock(i)
        return head

    def submit(self, i, typ, stream, evl, evs):
        self.now += 1
        c = self.c[i]
        seq = self._seq(c)
        op = seq[c["k"]]
        assert c["in_queue"] and op[0] == typ
        self.busy[stream] = max(self.now, self.busy[stream]) + op[2]
        self.done_at[(evl, evs)] = self.busy[stream]
        self.log.append("S %d %d %d %d %d %d" % (self.now, i, typ, stream, evl, evs))
        c["in_queue"] = False
        c["k"] += 1
        if c["k"] == len(seq):
            c["waiting"] = True
        else:
            c["next_push"] = self.now + seq[c["k"]][1]
        self._after_unlock(i)

    def query(self, evl, evs):
        self.now += 1
        done = self.now >= self.done_at.get((evl, evs), 0)
        self.log.append("Q %d %d %d %d" % (self.now, evl, evs, 1 if done else 0))
        return done

    def iter_lock(self, i):
        self._touch(i)

    def iter_done(self, i, it):
        self.c[i]["status"][it] = True
        self._after_unlock(i)

    def stop(self, k, locked):
        if not locked:
            self._touch(k)
        self.c[k]["stop_flag"] = True
        self.log.append("X %d %d" % (self.now, k))
        if not locked:
            self._after_unlock(k)


class Policy:
    def __init__(self, script, env):
        cl = script["clients"]
        self.n = len(cl)
        self.env = env
        self.max_sms = script["max_sms"]
        self.ops = [load_profile(c["profile"]) for c in cl]
        self.max_sms_clients = [max([o[3] for o in p] + [0]) for p in self.ops]
        self.is_train = [c["train"] for c in cl]
        self.num_kernels = [c["num_kernels"] for c in cl]
        self.max_iters = [c["num_iters"] for c in cl]
        self.seen = [0] * self.n
        self.event_ids = [0] * self.n
        self.cur_iters = [0] * self.n
        self.locked = [False] * self.n
        self.client_starts = [0] * self.n
        self.starts_set = [set() for _ in range(self.n)]
        self.penalty = 0

    def setup_change(self, i, path, num_kernels):
        self.ops[i] = load_profile(path)
        self.max_sms_clients[i] = max([o[3] for o in self.ops[i]] + [0])
        self.num_kernels[i] = num_kernels

    def _submit(self, typ, stream, idx, evid):
        if typ in UNSUPPORTED:
            raise RuntimeError("unsupported record")
        self.env.submit(idx, typ, stream, evid, self.event_ids[evid])
        if typ not in MEMOPS:
            self.event_ids[evid] += 1
            self.seen[idx] += 1

    def _reef(self, heads, depth):
        n, hp = self.n, self.n - 1
        if n == 1:
            if heads[0] >= 0:
                self._submit(heads[0], 0, 0, 0)
            return
        for i in range(n):
            if heads[i] >= 0 and (heads[i] == MALLOC or self.cur_iters[i] <= 10
                                  or self.cur_iters[hp] >= self.max_iters[hp]):
                self._submit(heads[i], i, i, i)
                return
        if heads[hp] >= 0:
            op1 = self.ops[hp][self.seen[hp]]
            self._submit(heads[hp], hp, hp, hp)
            for i in range(hp):
                if heads[i] >= 0:
                    op0 = self.ops[i][self.seen[i]]
                    if op0[4] <= op1[4] and op0[3] >= op1[3]:
                        self._submit(heads[i], i, i, i)
                        return
        else:
            self.penalty += sum(1 for i in range(hp) if heads[i] >= 0)
            if self.penalty >= depth:
                for i in range(hp):
                    if heads[i] >= 0:
                        self._submit(heads[i], i, i, i)
                self.penalty = 0

    def _sequential(self, heads, start):
        n, hp = self.n, self.n - 1
        if n == 1:
            if heads[0] >= 0:
                self._submit(heads[0], 0, 0, 0)
            return start
        if heads[hp] >= 0 and (self.cur_iters[hp] <= 10 or heads[hp] == MALLOC):
            self._submit(heads[hp], 0, hp, 0)
        for t in range(start + 1, start + n):
            i = t % (n - 1)
            if heads[i] >= 0 and (self.cur_iters[i] <= 10 or heads[i] == MALLOC):
                self._submit(heads[i], 0, i, 0)
                return t
        return start

    def run_phase(self, warmup, warmup_iters, reef, seq, depth, hp_limit, update_start):
        n, hp, env = self.n, self.n - 1, self.env
        profiles = [-1] * n
        large_found, total, start = False, 0, -1
        low, high = 0, self.max_sms_clients[0]
        thr = self.max_sms_clients[0] // 2
        hp_iter_duration = f32(0.0)
        hp_limit_f = f32(hp_limit)
        if not self.is_train[hp]:
            thr, update_start = self.max_sms, INT_MAX

        def fin(i):
            return (self.cur_iters[i] == self.max_iters[i] or (warmup and self.cur_iters[i] == warmup_iters)
                    or env.c[i]["stop_ack"])

        while True:
            size = 0
            heads = [-1] * n
            for i in range(n):
                if self.seen[i] == self.num_kernels[i]:
                    continue
                t = env.peek(i)
                if t >= 0:
                    heads[i] = t
                    if self.seen[i] == 0 and self.cur_iters[i] not in self.starts_set[i]:
                        self.client_starts[i] = env.now
                        self.starts_set[i].add(self.cur_iters[i])
            if reef:
                self._reef(heads, depth)
            elif seq:
                start = self._sequential(heads, start)
            else:
                if heads[hp] >= 0:
                    prof = self.ops[hp][self.seen[hp]][1]
                    self._submit(heads[hp], hp, hp, hp)
                    profiles[hp] = prof
                for t in range(start + 1, start + n):
                    j = t % (n - 1)
                    if heads[j] < 0:
                        continue
                    op = self.ops[j][self.seen[j]]
                    typ = heads[j]
                    memop = typ in MEMOPS
                    go = False
                    if self.seen[hp] == 0 or memop:
                        go = True
                    elif self.cur_iters[j] <= 10 or self.cur_iters[hp] >= self.max_iters[hp]:
                        go = True
                    elif self.seen[hp] >= update_start and op[3] <= thr and env.query(hp, update_start - 1):
                        go = True
                    elif self.seen[hp] > 0 and size + op[3] <= thr and (
                            op[1] == -1 or profiles[hp] == -1 or profiles[hp] != op[1]):
                        go = True
                    if go and large_found:
                        drained = True
                        for k in range(n - 1):
                            if self.event_ids[k] >= 1 and not env.query(k, self.event_ids[k] - 1):
                                drained = False
                                break
                        if drained:
                            large_found, total = False, 0
                        else:
                            go = False
                    if go:
                        size += op[3]
                        if not memop:
                            total = int(f32(total) + op[4])   # long += float
                        if total > depth and self.cur_iters[hp] < self.max_iters[hp]:
                            large_found = True
                        self._submit(typ, j, j, j)
                        start = j
            finished = 0
            for i in range(n):
                if fin(i):
                    finished += 1
                elif self.seen[i] == self.num_kernels[i]:
                    if not self.locked[i]:
                        env.iter_lock(i)
                        self.locked[i] = True
                    evl = 0 if seq else i
                    ready = True
                    if self.event_ids[evl] >= 1 and not env.query(evl, self.event_ids[evl] - 1):
                        ready = False
                    if ready:
                        self.seen[i] = 0
                        if seq:
                            self.event_ids[0] = 0
                        self.event_ids[i] = 0
                        env.iter_done(i, self.cur_iters[i])
                        self.cur_iters[i] += 1
                        self.locked[i] = False
                        duration = f32(env.now - self.client_starts[i])
                        duration = f32(np.float64(duration) / 1000.0)
                        if not reef and not seq and i == hp and self.is_train[hp]:
                            hp_iter_duration = f32(hp_iter_duration + duration)
                            if self.cur_iters[i] % 10 == 0 and low != thr:
                                avg = f32(np.float64(hp_iter_duration) / 10.0)
                                hp_iter_duration = f32(0.0)
                                if avg > hp_limit_f:
                                    high = thr
                                else:
                                    low = thr
                                thr = (low + high) // 2
                    if fin(i):
                        finished += 1
                        if not warmup and i == n - 1:
                            for k in range(n - 1):
                                env.stop(k, self.locked[k])
            if finished == n:
                return


def run_script(path):
    s = parse_script(path)
    env = Sim(s)
    pol = Policy(s, env)
    reef, seq = s["algo"] == "reef", s["algo"] == "sequential"
    for p, (warm, witers) in enumerate(s["phases"]):
        for c in env.c:
            c["limit"] = witers if warm else c["sc"]["num_iters"]
        pol.run_phase(warm, witers, reef, seq, s["depth"], s["hp_limit"], s["update_start"])
        env.log.append("E %d" % p)
        if p == 0:
            for i, c in enumerate(s["clients"]):
                if c["profile2"]:
                    pol.setup_change(i, c["profile2"], c["num_kernels2"])
    return "\n".join(env.log) + "\n"


if __name__ == "__main__":
    import sys
    text = run_script(sys.argv[1])
    print(hashlib.sha256(text.encode()).hexdigest(), text.count("\nS ") + text.startswith("S "))
