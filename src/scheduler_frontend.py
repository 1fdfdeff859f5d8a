"""Python front of the scheduler library: same class, method and argument order as
the reference's src/scheduler_frontend.py:8-35, so `launch_jobs.py` keeps working.

`run_scheduler` marshals the per-client lists into C arrays, calls `setup`, then
drives the three scheduling phases of the evaluation mode
(reference src/scheduler_frontend.py:68-94):

    barrier -> schedule(warm-up, 1 iteration) -> install second profiles
    barrier -> schedule(warm-up, 10 iterations)
    barrier -> schedule(measured run)
    barrier

Each client waits on the same barrier at start, after iteration 1, after
iteration 10 and at the end (reference benchmarking/benchmark_suite/train_imagenet.py:102,161-164,193-194,217).
Only the evaluation mode exists: the reference's other branch needs a
`scheduler.so` that its repository does not contain.
"""
import ctypes
import time

import torch


class PyScheduler:
    def __init__(self, sched_lib, num_clients):
        if torch.cuda.is_available():
            torch.cuda.set_device(torch.cuda.current_device())
        sched_lib.sched_init.restype = ctypes.c_void_p
        self._sched_lib = sched_lib
        self._num_clients = num_clients
        self._scheduler = ctypes.c_void_p(sched_lib.sched_init())
        self.total_time = None
        for name in ("orion_sched_client_stream",):
            if hasattr(sched_lib, name):
                getattr(sched_lib, name).restype = ctypes.c_void_p

    # -- helpers -----------------------------------------------------------
    def _sync(self):
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def client_stream(self, idx):
        """Raw cudaStream_t the scheduler created for client `idx` (valid after setup)."""
        return self._sched_lib.orion_sched_client_stream(self._scheduler, idx)

    def stats(self):
        out = (ctypes.c_ulonglong * 12)()
        self._sched_lib.orion_sched_stats(self._scheduler, out, 12)
        keys = ("polls", "hp_submits", "be_submits", "be_rejects", "queries", "join_timeouts", "max_sms", "green_be_sms",
                "forced_iter_ends", "quota_grants", "quota_ctas_sum", "clamped_launches")
        return dict(zip(keys, [int(v) for v in out]))

    def durations_ms(self, idx, cap=1 << 20):
        buf = (ctypes.c_float * cap)()
        n = self._sched_lib.orion_sched_durations(self._scheduler, idx, buf, cap)
        return [buf[i] for i in range(max(0, min(n, cap)))]

    def shutdown(self):
        self._sched_lib.orion_sched_shutdown(self._scheduler)

    def _schedule(self, num_clients, warmup, warmup_iters, reef, sequential, depth, hp_limit, update_start):
        self._sched_lib.schedule(self._scheduler, ctypes.c_int(num_clients), ctypes.c_bool(True), ctypes.c_int(0),
                                 ctypes.c_bool(warmup), ctypes.c_int(warmup_iters), ctypes.c_bool(reef),
                                 ctypes.c_bool(sequential), ctypes.c_int(depth), ctypes.c_int(hp_limit),
                                 ctypes.c_int(update_start))

    # -- the reference's entry point ---------------------------------------
    def run_scheduler(self, barriers, tids, model_names, kernel_files, additional_kernel_files, num_kernels,
                      additional_num_kernels, num_iters, profile, run_eval, reef, sequential, reef_depth, hp_limit,
                      update_start, train, on_setup=None):
        n = self._num_clients
        if len(tids) != n:
            raise ValueError("expected %d client thread ids, got %d" % (n, len(tids)))
        if not (run_eval and profile):
            raise NotImplementedError("only the evaluation mode (run_eval=True, profile=True) is available")

        int_array = ctypes.c_int * n
        str_array = ctypes.c_char_p * n
        bool_array = ctypes.c_bool * n
        # These arrays are borrowed by the library for the whole run: keep them on self.
        self._tids = int_array(*tids)
        self._num_kernels = int_array(*num_kernels)
        self._num_iters = int_array(*num_iters)
        self._models = str_array(*[m.encode("utf-8") for m in model_names])
        self._files = str_array(*[f.encode("utf-8") for f in kernel_files])
        self._train = bool_array(*[bool(t) for t in train])

        self._sched_lib.setup(self._scheduler, ctypes.c_int(n), self._tids, self._models, self._files, self._num_kernels,
                              self._num_iters, self._train, ctypes.c_bool(bool(reef)))
        if on_setup is not None:
            on_setup(self)

        args = (bool(reef), bool(sequential), int(reef_depth), int(hp_limit), int(update_start))
        barriers[0].wait()
        self._schedule(n, True, 1, *args)          # first iteration: warm-up and lazy initialisation
        self._sync()
        for j in range(n):                         # training clients launch a different op sequence from iteration 1 on
            if additional_kernel_files[j] is not None:
                self._sched_lib.setup_change(self._scheduler, ctypes.c_int(j), additional_kernel_files[j].encode("utf-8"),
                                             ctypes.c_int(additional_num_kernels[j]))
        barriers[0].wait()
        self._schedule(n, True, 10, *args)         # warm-up until every client has done 10 iterations
        self._sync()
        barriers[0].wait()
        start = time.time()
        self._schedule(n, False, 0, *args)         # measured run
        self.shutdown()                            # late calls of the clients (result read-back) run unscheduled
        barriers[0].wait()
        self._sync()
        self.total_time = time.time() - start
        print("Total time is %f" % self.total_time)
