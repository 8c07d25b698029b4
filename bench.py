"""Benchmark of the flash_dism hard path (labels -> forward -> backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the whole path over one batch of the training shape (B8 H16 N8192 D64 R32
DV64, 512 symbols per head): the discretiser for q and k, the fused hard forward, and the hard
backward.  Metric: query positions per second, whole job.  With N > 1 (torchrun, one rank per GPU)
the SAME problem is split over the ranks by heads (16 / N heads per GPU: heads are independent, so
there is no collective on the data path; strong scaling) and the time is the maximum over ranks.

`value` is timed with the inputs resident in HBM; `e2e` times the same step through the drop-in
Python API with pinned host inputs copied in and results copied out inside the timed region.
`--impl reference` times the CPU restatement of the reference's dense algorithm (plus the
reference's own native CPU forward when it was built) on a bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPE = dict(batch=8, heads=16, n=8192, d=64, r=32, dv=64, vocab=512)
WORKLOAD = 'training shape B{batch} H16 N8192 D64 R32 DV64 V512, all rows hard, tau 0.5: labels(q), labels(k), hard forward, hard backward'
# Algorithmic bytes per query position of each kernel launch (inputs read once, outputs written once).
KERNEL_BYTES = {
    'labels_pair': 264,          # q and k in one launch: two bf16 rows of 64 read, two labels written
    'hard_forward': 396,         # labels 8, sq+sk 128, v 128 read; out 128, lse2 4 written
    'hard_backward_query': 524,  # sq,sk 128, v,dO 256, labels 8, lse2 4 read; dsq (f32) 128 written
    'hard_backward_key': 588,    # the same reads; dsk 64, dv 128 written
    'hard_backward': 524 + 588,  # both passes in one launch, which the library does when a GPU holds little work
}
STEP_BYTES = 2 * 132 + 396 + 716  # whole path: two label launches, forward, backward (inputs counted once)


def measured_traffic():
    """dram__bytes_read.sum + dram__bytes_write.sum per launch at the benchmark batch on one GPU, as captured with
    ncu (profiles/traffic_B8.json, with the command that made it); None for kernels without a capture."""
    path = os.path.join(ROOT, 'profiles', 'traffic_B8.json')
    if not os.path.exists(path):
        return {}
    with open(path) as f:
        return json.load(f).get('bytes_per_launch', {})


def measured_peak(key='hbm_gbs', fallback=6650.0):
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)[key]), 'measured'
    return fallback, 'fallback'


# The discretiser is the one contraction on the path: 2 * D * V flops per row and side.  Its bound is the tensor pipe
# (burst bf16 figure: the kernel runs 0.3 ms at full clocks, not seconds under the power cap); every other kernel moves bytes.
KERNEL_FLOPS = {'labels_pair': 2 * 2 * 64 * 512}


def kernel_roofline(name, ms, positions, traffic):
    """achieved / peak of one kernel launch over `positions` query positions that took `ms`."""
    if name in KERNEL_FLOPS:
        peak, kind = measured_peak('bf16_tflops', 1590.0)
        achieved = KERNEL_FLOPS[name] * positions / (ms * 1e-3) / 1e12
        return {'bound': 'tensor', 'kernel': name, 'achieved': achieved, 'peak': peak, 'unit': 'TFLOP/s', 'frac': achieved / peak,
                'peak_kind': kind, 'traffic': traffic, 'algorithmic_flops_per_launch': KERNEL_FLOPS[name] * positions,
                'algorithmic_bytes_per_launch': KERNEL_BYTES[name] * positions}
    peak, kind = measured_peak()
    achieved = KERNEL_BYTES[name] * positions / (ms * 1e-3) / 1e9
    return {'bound': 'hbm', 'kernel': name, 'achieved': achieved, 'peak': peak, 'unit': 'GB/s', 'frac': achieved / peak,
            'peak_kind': kind, 'traffic': traffic, 'algorithmic_bytes_per_launch': KERNEL_BYTES[name] * positions}


def bind_to_gpu_cpus(index):
    """Runs this process on the CPUs next to GPU `index` (NVML's CPU affinity of the device), so that the pinned host
    buffers of the end-to-end leg, which are placed where the allocating thread runs, sit on the GPU's own NUMA node.
    Returns (the previous CPU set, a note for the JSON line); nothing changes when NVML cannot say."""
    before = os.sched_getaffinity(0)
    try:
        import pynvml
        pynvml.nvmlInit()
        properties = torch.cuda.get_device_properties(index)
        try:
            handle = pynvml.nvmlDeviceGetHandleByUUID('GPU-' + str(properties.uuid))
        except Exception:
            handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        near = {cpu for cpu in before if (words[cpu // 64] >> (cpu % 64)) & 1}
        if near and near != before:
            os.sched_setaffinity(0, near)
            return before, f'{len(near)} of {len(before)} CPUs: those next to the GPU'
        return before, f'all {len(before)} CPUs (already next to the GPU)'
    except Exception as error:
        return before, f'all {len(before)} CPUs (NVML affinity unavailable: {type(error).__name__})'


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index):
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self.stop = threading.Event()
        self.thread = threading.Thread(target=self.run, daemon=True)

    def run(self):
        query = ('clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
                 'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')
        names = ('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap')
        while not self.stop.is_set():
            try:
                line = subprocess.run(['nvidia-smi', f'--id={self.index}', f'--query-gpu={query}',
                                       '--format=csv,noheader,nounits'], capture_output=True, text=True,
                                      timeout=5).stdout.strip().split(',')
                self.samples.append(float(line[0]))
                self.max_mhz = float(line[1])
                for name, value in zip(names, line[2:]):
                    if value.strip().lower().startswith('active'):
                        self.reasons.add(name)
            except Exception:
                pass
            self.stop.wait(.1)

    def __enter__(self):
        self.thread.start()
        return self

    def __exit__(self, *exc):
        self.stop.set()
        self.thread.join()

    def summary(self):
        return dict(sm_mhz=float(np.median(self.samples)) if self.samples else None, sm_max_mhz=self.max_mhz,
                    reasons=sorted(self.reasons))


def make_inputs(seed, device, rank=0, world=1):
    """Host (pinned) and device operands of this rank: the whole problem is drawn from one seed on every
    rank, then cut to the rank's contiguous slice of heads (dism_b200/sharding.py)."""
    from dism_b200.sharding import shard_operands
    s = SHAPE
    g = torch.Generator().manual_seed(seed)
    shape = (s['batch'], s['n'], s['heads'])
    host = {}
    host['q'], host['k'] = [torch.randn(*shape, s['d'], generator=g).bfloat16() for _ in range(2)]
    host['v'] = torch.randn(*shape, s['dv'], generator=g).bfloat16()
    host['sq'], host['sk'] = [(torch.nn.functional.silu(torch.randn(*shape, s['r'], generator=g)) * .4).bfloat16()
                              for _ in range(2)]
    params = {name: torch.nn.functional.silu(torch.randn(s['heads'], s['vocab'], s['d'], generator=g)).bfloat16()
              for name in ('eq', 'ek')}
    host['dout'] = torch.randn(*shape, s['dv'], generator=g).bfloat16()
    params['tau'] = torch.full((s['heads'],), .5)
    params['hard'] = torch.ones(s['batch'], s['heads'], dtype=torch.bool)
    mine = shard_operands({**host, **params}, rank, world)
    host = {k: mine[k].pin_memory() for k in host}
    return host, {k: mine[k].to(device) for k in params}


def run_ours(args):
    import torch.distributed as dist
    import dism_b200
    dism_b200.install_dropin()
    import cu_flash_dism as cu
    from flash_dism.hard_forward import forward_hard, hard_readout, hard_log_weights
    from flash_dism.hard_backward import backward_hard

    rank, world = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1))
    local = int(os.environ.get('LOCAL_RANK', 0))
    torch.cuda.set_device(local)
    device = torch.device('cuda', local)
    if world > 1:
        dist.init_process_group('nccl', device_id=device)
    s = SHAPE
    if s['heads'] % world:
        raise SystemExit(f"{s['heads']} heads do not split evenly over {world} GPUs")
    split = args.share if args.kernels_only and args.share else world  # --share: rank 0's slice of a wider split, alone
    heads_here = s['heads'] // split
    total_positions = s['batch'] * s['heads'] * s['n']  # the whole job, over all ranks
    positions = s['batch'] * heads_here * s['n']        # this rank's share
    all_cpus, cpu_note = bind_to_gpu_cpus(local)
    host, params = make_inputs(0, device, rank, split)
    resident = {k: v.to(device) for k, v in host.items()}
    launches = [0]

    def step(x, stage_events=None):
        mark = (lambda: None) if stage_events is None else (lambda: stage_events.append(_event()))
        mark()
        iq, ik = cu.labels_pair(x['q'], params['eq'], x['k'], params['ek'])
        mark()
        lut = hard_log_weights(params['tau'], s['n'])  # built once per step, as forward_hard(save_state=True) keeps it for the backward
        out, norm = hard_readout(x['sq'], x['sk'], x['v'], iq, ik, params['hard'], None, lut)
        mark()
        grads = backward_hard(x['sq'], x['sk'], x['v'], x['dout'], iq, ik, params['hard'], norm,
                              dict(boundary=None, log_weights=lut))
        mark()
        # labels of q and k (one launch); log weights; readout: index, tiles, label-block kernel, dense-route kernel (its
        # CTAs return at once on these labels); backward: tiles of both passes with the dlog table (one launch),
        # query-major and key-major pass (one launch when the GPU holds at most 262144 positions), dense-route kernel, tau
        # reduction (the index is the readout's)
        launches[0] += 1 + 1 + 4 + (4 if positions <= 262144 else 5)
        return out, norm, grads

    def _event():
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # A rank's inputs of one step must not sit in the 126 MB L2 when the step starts.  With few heads per GPU they
    # would: then a 256 MB write flushes L2 before every step and the steps are timed one by one (the flush is not
    # part of any step's time).
    flush = sum(v.numel() * v.element_size() for v in resident.values()) < 2 * 126e6
    scrub = torch.empty(256 << 20, dtype=torch.uint8, device=device) if flush else None
    for _ in range(args.warmup):
        step(resident)
    # With that little work per GPU a step's ten launches take the host longer than the GPU takes to run them, and the
    # host would set the pace.  The step is then captured once into a CUDA graph (the drop-in's calls, allocations
    # included, as a training loop with static shapes would capture them) and every timed step is one replay.
    graph = None
    if flush:
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            graph_outputs = step(resident)  # kept: the graph writes its results here on every replay
        for _ in range(args.warmup):
            graph.replay()
    barrier()
    launches[0] = 0
    launches_per_step = 1 + 1 + 4 + (4 if positions <= 262144 else 5)
    stages, replays = [], []
    with ClockSampler(local) as clocks:
        start = _event()
        for index in range(args.steps):
            if flush:
                scrub.fill_(index & 255)
                before = _event()
                graph.replay()
                replays.append((before, _event()))
                launches[0] += launches_per_step
            else:
                events = []
                step(resident, events)
                stages.append(events)
        stop = _event()
        barrier()
        elapsed_ms = sum(a.elapsed_time(b) for a, b in replays) if flush else start.elapsed_time(stop)
        kernel_launches = launches[0]
        if flush:  # the stages of a step, from eager steps outside the timed region (events cannot be timed inside a graph)
            for _ in range(args.warmup):  # (the capture emptied the allocator's cache: let it fill again first)
                step(resident)
            for index in range(args.steps):
                scrub.fill_(index & 255)
                events = []
                step(resident, events)
                stages.append(events)
            torch.cuda.synchronize()
        stage_ms = np.array([[a.elapsed_time(b) for a, b in zip(e, e[1:])] for e in stages]).mean(0)

        # per-kernel device times: K more steps with the library's event timing switched on
        from dism_b200 import _lib
        _lib.load().dism_profile_enable(1)
        for _ in range(args.steps):
            step(resident)
        torch.cuda.synchronize()
        kernel_ms = {}
        for name, ms in _lib.kernel_timings():
            kernel_ms.setdefault(name, []).append(ms)
        _lib.load().dism_profile_enable(0)
        kernel_ms = {name: float(np.mean(v)) for name, v in kernel_ms.items()}
        if args.kernels_only:
            if rank == 0:
                print(json.dumps({'profiling_case': True, 'batch': s['batch'], 'ms_per_step': elapsed_ms / args.steps,
                                  'stage_ms': dict(zip(('labels', 'forward', 'backward'), map(float, stage_ms))),
                                  'kernel_ms': kernel_ms}))
            return
        # end to end: every step copies its inputs from pinned host memory and all of its results back.
        # Steps are pipelined over three streams (copy in, compute, copy out) with three buffer sets, as a
        # training loop that prefetches its next batch would do; the timed region covers all of it,
        # including the first copy in and the last copy out, which overlap with nothing: enough steps are
        # run for that fill and drain to weigh a few per cent.
        copy_names = ('q', 'k', 'sq', 'sk', 'v', 'dout')
        h2d = sum(host[k].numel() * host[k].element_size() for k in copy_names)
        copy_in, compute, copy_out = (torch.cuda.Stream(device) for _ in range(3))
        slots = 3
        staged = [{k: torch.empty_like(resident[k]) for k in copy_names} for _ in range(slots)]
        results = [None] * slots
        result_host = [None] * slots
        ready_in = [torch.cuda.Event() for _ in range(slots)]
        done_compute = [torch.cuda.Event() for _ in range(slots)]
        done_out = [torch.cuda.Event() for _ in range(slots)]
        d2h = [0]

        def e2e_step(index):
            slot = index % slots
            with torch.cuda.stream(copy_in):
                copy_in.wait_event(done_compute[slot])  # the previous user of this input buffer has finished
                for k in copy_names:
                    staged[slot][k].copy_(host[k], non_blocking=True)
                ready_in[slot].record(copy_in)
            with torch.cuda.stream(compute):
                compute.wait_event(ready_in[slot])
                compute.wait_event(done_out[slot])  # the previous results of this slot have left the device
                out, norm, grads = step(staged[slot])
                results[slot] = [out, norm, *grads]
                done_compute[slot].record(compute)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(done_compute[slot])
                if result_host[slot] is None:
                    result_host[slot] = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in results[slot]]
                for dst, src in zip(result_host[slot], results[slot]):
                    dst.copy_(src, non_blocking=True)
                    src.record_stream(copy_out)
                done_out[slot].record(copy_out)
            d2h[0] = sum(o.numel() * o.element_size() for o in results[slot])

        for index in range(2 * slots):
            e2e_step(index)
        barrier()
        e2e_steps = max(24, 3 * args.steps)
        e2e_start = torch.cuda.Event(enable_timing=True)
        e2e_stop = torch.cuda.Event(enable_timing=True)
        e2e_start.record(torch.cuda.current_stream())
        for stream in (copy_in, compute, copy_out):
            stream.wait_event(e2e_start)
        for index in range(e2e_steps):
            e2e_step(index)
        for stream in (copy_in, compute, copy_out):
            torch.cuda.current_stream().wait_stream(stream)
        e2e_stop.record(torch.cuda.current_stream())
        barrier()
        e2e_ms = e2e_start.elapsed_time(e2e_stop)
        d2h = d2h[0]

    os.sched_setaffinity(0, all_cpus)  # the CPU baseline below runs on every host core
    flip_rate = label_flip_rate(cu, resident, params)
    long_context = long_context_record(cu, forward_hard, device, rank, world, args)
    times = torch.tensor([elapsed_ms, e2e_ms, long_context['ms_labels'] + long_context['ms_forward']], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, long_ms = times.tolist()
    long_context['value'] = long_context['positions_per_gpu'] * world / (long_ms * 1e-3)  # all ranks' heads over the slowest rank's time
    if rank == 0:
        peak, peak_kind = measured_peak()
        ms_per_step = elapsed_ms / args.steps
        dominant = max(KERNEL_BYTES, key=lambda name: kernel_ms.get(name, 0.))
        captured = measured_traffic() if world == 1 and s['batch'] == 8 else {}
        roofline = kernel_roofline(dominant, kernel_ms[dominant], positions, captured.get(dominant))
        # the other hot kernels beside it, and the whole step against the HBM peak
        roofline['kernels'] = {name: {k: v for k, v in kernel_roofline(name, kernel_ms[name], positions, captured.get(name)).items()
                                      if k in ('bound', 'achieved', 'unit', 'frac', 'traffic')}
                               for name in KERNEL_BYTES if name in kernel_ms}
        roofline['whole_step_frac'] = STEP_BYTES * positions / (ms_per_step * 1e-3) / 1e9 / peak
        line = {
            'metric': 'DISM fwd+bwd query-positions/s (labels + hard forward + hard backward)',
            'value': total_positions / (ms_per_step * 1e-3), 'unit': 'positions/s', 'n_gpus': world,
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': ms_per_step, 'higher_is_better': True,
            'scaling': 'strong', 'vs_baseline': None, 'dtype': 'bf16 vectors, int32 labels, f32 accumulate',
            'data': 'synthetic (seeded N(0,1) q,k,v,dO; silu(N(0,1)) codebooks and readout features)',
            'config': {'workload': WORKLOAD.format(batch=s['batch']),
                       'parallelism': f'16 heads / {world} = {heads_here} heads per GPU, one problem, no collective',
                       'l2': f'inputs per step and GPU ({sum(v.numel() * v.element_size() for v in host.values()) / 1e6:.0f} MB) '
                             + ('exceed L2' if not flush else 'are flushed from L2 by a 256 MB write between steps; each step is one replay of a CUDA graph of the step'),
                       'host_cpus': cpu_note},
            'stage_ms': {'labels': float(stage_ms[0]), 'forward': float(stage_ms[1]), 'backward': float(stage_ms[2])},
            'kernel_ms': kernel_ms,
            'per_gpu_value': positions / (ms_per_step * 1e-3),
            'e2e': {'value': total_positions / (e2e_ms / e2e_steps * 1e-3), 'unit': 'positions/s',
                    'h2d_bytes_per_step': h2d, 'd2h_bytes_per_step': d2h, 'steps': e2e_steps},
            'gpu_launches': kernel_launches,
            'clocks': clocks.summary(),
            'roofline': roofline,
            'label_flip_rate': flip_rate,
            'long_context': long_context,
            'cpu_baseline': cpu_baseline() if world == 1 else None,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def label_flip_rate(cu, x, params):
    """Share of this rank's labels (q and k, benchmark data) that differ from torch.argmax of the FP32 einsum: the
    kernel's labels are defined by a pinned FP32 summation order, the einsum's by cuBLAS; only near ties can differ."""
    differing, total = 0, 0
    for rows, codes in ((x['q'], params['eq']), (x['k'], params['ek'])):
        mine = cu.labels(rows, codes)
        for head in range(codes.size(0)):
            logits = torch.einsum('bnd,vd->bnv', rows[:, :, head].float(), codes[head].float())
            differing += int((logits.argmax(-1).int() != mine[:, head]).sum())
            total += mine[:, head].numel()
    return differing / total


def long_context_record(cu, forward_hard, device, rank, world, args):
    """The long-context workload on this rank: forward only on 4 heads of B1 H32 N131072 D64 R32 DV64 (with 8 ranks
    that is the whole workload; with fewer, each rank still takes 4 heads).  Every 4096 positions the q rows of a
    random 1024-long window repeat the k rows of an earlier window, which forces 1024-long label runs.  Rank 0
    checks one head against the reference's own native CPU forward (oracle/_ref), all 131072 rows."""
    from dism_b200 import _lib
    b, h, n, d, r, dv, vocab = 1, 4, 131072, 64, 32, 64, 512
    g = torch.Generator(device=device).manual_seed(100 + rank)
    k = torch.randn(b, n, h, d, generator=g, device=device).bfloat16()
    q = torch.randn(b, n, h, d, generator=g, device=device).bfloat16()
    rng = np.random.default_rng(100 + rank)
    for start in range(4096, n, 4096):
        target = start + int(rng.integers(0, 3072))
        source = int(rng.integers(0, target - 1024))
        q[:, target:target + 1024] = k[:, source:source + 1024]
    codebook = torch.nn.functional.silu(torch.randn(h, vocab, d, generator=g, device=device)).bfloat16()
    sq, sk = [(torch.nn.functional.silu(torch.randn(b, n, h, r, generator=g, device=device)) * .4).bfloat16() for _ in range(2)]
    v = torch.randn(b, n, h, dv, generator=g, device=device).bfloat16()
    hard, tau = torch.ones(b, h, dtype=torch.bool, device=device), torch.full((h,), .05, device=device)

    def timed(fn):
        for _ in range(max(1, args.warmup)):
            fn()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(args.steps):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / args.steps

    iq, ik = cu.labels_pair(q, codebook, k, codebook)  # one shared codebook, so repeated rows get equal labels
    ms_labels = timed(lambda: cu.labels_pair(q, codebook, k, codebook))
    ms_forward = timed(lambda: forward_hard(sq, sk, v, iq, ik, hard, tau))
    _lib.load().dism_profile_enable(1)
    out, norm = forward_hard(sq, sk, v, iq, ik, hard, tau)
    torch.cuda.synchronize()
    kernel_ms = dict(_lib.kernel_timings())
    _lib.load().dism_profile_enable(0)
    record = {'workload': 'long context forward: 4 heads per GPU of B1 H32 N131072 D64 R32 DV64 V512, planted 1024-long runs, tau 0.05',
              'metric': 'query positions/s (labels + hard forward)', 'positions_per_gpu': b * h * n, 'ms_labels': ms_labels,
              'ms_forward': ms_forward, 'kernel_ms': kernel_ms, 'max_log2_normaliser': float(norm.max()), 'parity': None}
    if rank == 0:
        from oracle import dism_oracle
        if dism_oracle.reference_lib() is None:
            record['parity'] = 'not checked: oracle/_ref (the reference native CPU forward) was not built'
        else:
            f = lambda t: t[0, :, 0].float().cpu().numpy()
            want = dism_oracle.reference_forward_many(f(sq)[None], f(sk)[None], f(v)[None], iq[0, 0].cpu().numpy()[None],
                                                      ik[0, 0].cpu().numpy()[None], np.full(1, .05), threads=1)[0]
            error = np.abs(out[0, :, 0].float().cpu().numpy() - want)
            bound = .008 + .025 * np.abs(want)  # the forward tests' tolerance
            record['parity'] = {'against': 'reference native CPU forward (Builder + execute<float>), head 0, all 131072 rows',
                                'max_abs_error': float(error.max()), 'rows_outside_tolerance': int((error > bound).any(-1).sum())}
    return record


def cpu_inputs(heads, seed=0):
    """Synthetic operands of `heads` (batch, head) slices of the benchmark shape, as numpy arrays."""
    from oracle import dism_oracle as o
    s = SHAPE
    rng = np.random.default_rng(seed)
    b, n = 1, s['n']
    f = lambda *shape: o.bf16_round(rng.standard_normal(shape).astype(np.float32))
    silu = lambda x: o.bf16_round((x / (1 + np.exp(-x))).astype(np.float32))
    return dict(q=f(b, n, heads, s['d']), k=f(b, n, heads, s['d']),
                eq=silu(rng.standard_normal((heads, s['vocab'], s['d']))),
                ek=silu(rng.standard_normal((heads, s['vocab'], s['d']))),
                sq=silu(rng.standard_normal((b, n, heads, s['r']))) * np.float32(.5),
                sk=silu(rng.standard_normal((b, n, heads, s['r']))) * np.float32(.5),
                v=f(b, n, heads, s['dv']), dout=f(b, n, heads, s['dv']),
                tau=np.full(heads, .5, np.float32), hard=np.ones((b, heads), bool))


def cpu_sample(x, threads):
    """Time the CPU path on prepared operands; returns seconds per stage (inputs are not timed).  The forward leg runs
    the reference's own native CPU forward (its planner and executor in float32, one (batch, head) sequence per task
    on `threads` host threads) when oracle/_ref was built, else the C port; labels and backward are the port."""
    from oracle import dism_oracle as o
    # the discretiser on the CPU side is a plain fp32 GEMM + argmax (what the reference's torch path does)
    t0 = time.perf_counter()
    torch.set_num_threads(threads)
    iq = torch.argmax(torch.einsum('bnhd,hvd->bnhv', torch.from_numpy(x['q']), torch.from_numpy(x['eq'])), -1)
    ik = torch.argmax(torch.einsum('bnhd,hvd->bnhv', torch.from_numpy(x['k']), torch.from_numpy(x['ek'])), -1)
    iq, ik = [t.transpose(1, 2).contiguous().int().numpy() for t in (iq, ik)]
    t1 = time.perf_counter()
    native = o.reference_lib() is not None
    if native:
        per_head = lambda a: np.ascontiguousarray(a[0].transpose(1, 0, 2))  # [N,H,C] -> [H,N,C]
        o.reference_forward_many(per_head(x['sq']), per_head(x['sk']), per_head(x['v']), iq[0], ik[0],
                                 x['tau'].astype(np.float64), threads=threads)
    else:
        o.forward(x['sq'], x['sk'], x['v'], iq, ik, x['hard'], x['tau'], threads=threads)
    t2 = time.perf_counter()
    o.backward(x['sq'], x['sk'], x['v'], x['dout'], iq, ik, x['hard'], x['tau'], threads=threads)
    t3 = time.perf_counter()
    return dict(labels=t1 - t0, forward=t2 - t1, backward=t3 - t2), native


def cpu_legs(native):
    return {'labels': 'port (torch fp32 GEMM + argmax)',
            'forward': 'reference (native planner + execute<float>)' if native else 'port (C restatement of the dense recurrence)',
            'backward': 'port (C restatement of the dense recurrence; the reference has no native CPU backward)'}


def cpu_baseline(heads=None):
    cores = os.cpu_count() or 1
    heads = heads or min(128, 4 * max(cores, 8))
    cpu_sample(cpu_inputs(2), cores)  # warm caches and the thread pool
    t, native = cpu_sample(cpu_inputs(heads), cores)
    total = t['labels'] + t['forward'] + t['backward']
    return {'value': heads * SHAPE['n'] / total, 'unit': 'positions/s', 'cores': cores, 'kind': 'reference' if native else 'port',
            'legs': cpu_legs(native),
            'sample': f'{heads} of the 128 (batch, head) slices at N=8192, one slice per task on all {cores} host threads',
            'seconds': t}


def run_reference(args):
    rank = int(os.environ.get('RANK', 0))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    heads = min(128, 4 * max(cores, 8))
    small, inputs = cpu_inputs(2), cpu_inputs(heads)
    for _ in range(args.warmup):
        cpu_sample(small, cores)
    elapsed, native, seconds = 0., False, {}
    for step in range(args.steps):
        t, native = cpu_sample(inputs, cores)
        elapsed += t['labels'] + t['forward'] + t['backward']
        seconds = {k: seconds.get(k, 0.) + v / args.steps for k, v in t.items()}
    value = heads * SHAPE['n'] * args.steps / elapsed
    base = {'value': value, 'unit': 'positions/s', 'cores': cores, 'kind': 'reference' if native else 'port', 'legs': cpu_legs(native),
            'sample': f'each step = {heads} of the 128 (batch, head) slices at N=8192, one slice per task on all {cores} host threads',
            'seconds': seconds}
    print(json.dumps({
        'impl': 'reference', 'metric': 'DISM fwd+bwd query-positions/s (labels + hard forward + hard backward)',
        'value': value, 'unit': 'positions/s', 'n_gpus': int(os.environ.get('WORLD_SIZE', 1)), 'steps': args.steps,
        'warmup': args.warmup, 'ms_per_step': elapsed / args.steps * 1e3, 'higher_is_better': True, 'scaling': 'strong',
        'vs_baseline': None, 'dtype': 'f32 (reference forward), f64 accumulate over bf16-rounded f32 inputs (port)', 'data': 'synthetic',
        'config': {'workload': WORKLOAD.format(batch=SHAPE['batch']),
                   'sample': f'{heads} of the 128 (batch, head) slices per step on the host cores'},
        'cpu_baseline': base,
        'e2e': {'value': value, 'unit': 'positions/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0}}))


def run_other_workload(args):
    """The side workloads: forward only on the long-context shape (one GPU's share: 4 heads of
    N = 131072 with planted 1024-long runs), forward and backward on dense labels, the integer stages of the saved-state
    route, a pack of documents, and the single-longest-match reduction on symbol streams."""
    import dism_b200
    dism_b200.install_dropin()
    import cu_flash_dism as cu
    from flash_dism.hard_forward import forward_hard
    torch.cuda.set_device(0)
    g = torch.Generator(device='cuda').manual_seed(0)

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(args.steps):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / args.steps

    if args.workload == 'long_context':
        b, h, n, d, r, dv, vocab = 1, 4, 131072, 64, 32, 64, 512
        k = torch.randn(b, n, h, d, generator=g, device='cuda').bfloat16()
        q = torch.randn(b, n, h, d, generator=g, device='cuda').bfloat16()
        rng = np.random.default_rng(0)
        for start in range(4096, n, 4096):  # queries of a window repeat the keys of an earlier window
            target = start + int(rng.integers(0, 3072))
            source = int(rng.integers(0, target - 1024))
            q[:, target:target + 1024] = k[:, source:source + 1024]
        codebook = torch.nn.functional.silu(torch.randn(h, vocab, d, generator=g, device='cuda')).bfloat16()
        sq, sk = [(torch.nn.functional.silu(torch.randn(b, n, h, r, generator=g, device='cuda')) * .4).bfloat16()
                  for _ in range(2)]
        v = torch.randn(b, n, h, dv, generator=g, device='cuda').bfloat16()
        hard, tau = torch.ones(b, h, dtype=torch.bool, device='cuda'), torch.full((h,), .05, device='cuda')
        iq, ik = cu.labels_pair(q, codebook, k, codebook)  # one shared codebook, so copied rows match
        ms_labels = timed(lambda: cu.labels_pair(q, codebook, k, codebook))
        ms_forward = timed(lambda: forward_hard(sq, sk, v, iq, ik, hard, tau))
        from dism_b200 import _lib
        _lib.load().dism_profile_enable(1)
        _, norm = forward_hard(sq, sk, v, iq, ik, hard, tau)
        torch.cuda.synchronize()
        kernel_ms = dict(_lib.kernel_timings())
        _lib.load().dism_profile_enable(0)
        print(json.dumps({'workload': 'long context forward, B1 H4 N131072 (one GPU of eight), planted 1024-long runs',
                          'metric': 'query positions/s', 'value': b * h * n / ((ms_labels + ms_forward) * 1e-3),
                          'ms_labels': ms_labels, 'ms_forward': ms_forward, 'kernel_ms': kernel_ms,
                          'max_log2_normaliser': float(norm.max()),
                          'steps': args.steps, 'warmup': args.warmup}))
    elif args.workload == 'dense_labels':
        # the shape of the reference's own hard-forward benchmark (dism_v3/tools/bench_hard_forward.py:18: B16 N2048 H6 R32
        # DV64, tau .5, labels uniform over 512 symbols or all equal), fixed layout: complete forward and backward
        from flash_dism.hard_forward import hard_log_weights
        from flash_dism.hard_backward import backward_hard
        b, n, h, r, dv = 16, 2048, 6, 32, 64
        sq, sk = [(torch.randn(b, n, h, r, generator=g, device='cuda') * .3).bfloat16() for _ in range(2)]
        v, dout = [torch.randn(b, n, h, dv, generator=g, device='cuda').bfloat16() for _ in range(2)]
        hard, tau = torch.ones(b, h, dtype=torch.bool, device='cuda'), torch.full((h,), .5, device='cuda')
        record = {'workload': 'hard forward and backward, B16 N2048 H6 R32 DV64, labels over 512 symbols or all equal', 'ms': {}}
        for pattern in ('equal', 'random'):
            iq, ik = [torch.randint(0, 512, (b, h, n), generator=g, device='cuda', dtype=torch.int32) for _ in range(2)]
            if pattern == 'equal':
                iq.zero_(), ik.zero_()
            _, norm = forward_hard(sq, sk, v, iq, ik, hard, tau)
            lut = hard_log_weights(tau, n)
            record['ms'][pattern] = {
                'forward': timed(lambda: forward_hard(sq, sk, v, iq, ik, hard, tau)),
                'backward': timed(lambda: backward_hard(sq, sk, v, dout, iq, ik, hard, norm, dict(boundary=None, log_weights=lut)))}
        record.update(steps=args.steps, warmup=args.warmup)
        print(json.dumps(record))
    elif args.workload == 'packed':
        # The benchmark's tokens as one pack: 8 training rows of 8192 tokens, each cut into 256-aligned documents of random
        # lengths, 16 heads, R32 DV64, labels uniform over 512 symbols.  Forward and backward with the layout, beside the
        # same tensors run as 8 whole sequences (fixed layout).  A document sees only itself, so the pack has fewer pairs.
        from flash_dism.hard_forward import hard_log_weights
        from flash_dism.hard_backward import backward_hard
        from flash_dism.varlen import VarlenLayout
        rows, row_tokens, h, r, dv = 8, 8192, 16, 32, 64
        n = rows * row_tokens
        rng = np.random.default_rng(0)
        offsets = [0]
        for row in range(rows):
            at = 0
            while at < row_tokens:
                at = min(row_tokens, at + 256 * int(rng.integers(1, 17)))
                offsets.append(row * row_tokens + at)
        layout = VarlenLayout.from_cu_seqlens(torch.tensor(offsets, dtype=torch.int32), n)
        sq, sk = [(torch.randn(1, n, h, r, generator=g, device='cuda') * .3).bfloat16() for _ in range(2)]
        v, dout = [torch.randn(1, n, h, dv, generator=g, device='cuda').bfloat16() for _ in range(2)]
        iq, ik = [torch.randint(0, 512, (1, h, n), generator=g, device='cuda', dtype=torch.int32) for _ in range(2)]
        hard, tau = torch.ones(rows, h, dtype=torch.bool, device='cuda'), torch.full((h,), .5, device='cuda')
        lut = hard_log_weights(tau, row_tokens)
        _, norm = forward_hard(sq, sk, v, iq, ik, hard, tau, layout=layout)
        record = {'workload': f'one pack of {len(offsets) - 1} documents in 8 rows of 8192 tokens, H16 R32 DV64, beside the same tokens as 8 whole sequences',
                  'ms': {'packed': {
                      'forward': timed(lambda: forward_hard(sq, sk, v, iq, ik, hard, tau, layout=layout)),
                      'forward keeping the rectangle': timed(lambda: forward_hard(sq, sk, v, iq, ik, hard, tau, layout=layout, save_state=True)),
                      'backward': timed(lambda: backward_hard(sq, sk, v, dout, iq, ik, hard, norm, dict(boundary=None, log_weights=lut),
                                                              layout=layout))}}}
        fixed = [t.view(rows, row_tokens, h, -1) for t in (sq, sk, v, dout)]
        fq, fk = [t.view(h, rows, row_tokens).transpose(0, 1).contiguous() for t in (iq, ik)]
        _, fixed_norm = forward_hard(*fixed[:3], fq, fk, hard, tau)
        record['ms']['whole sequences'] = {
            'forward': timed(lambda: forward_hard(*fixed[:3], fq, fk, hard, tau)),
            'forward keeping the rectangle': timed(lambda: forward_hard(*fixed[:3], fq, fk, hard, tau, save_state=True)),
            'backward': timed(lambda: backward_hard(*fixed[:3], fixed[3], fq, fk, hard, fixed_norm, dict(boundary=None, log_weights=lut)))}
        record.update(steps=args.steps, warmup=args.warmup)
        print(json.dumps(record))
    elif args.workload == 'saved_state':
        # The integer stages that forward_hard(save_state=True) adds: strip summaries, then boundary composition, on the
        # benchmark shape and on the shape of the reference's own hard-forward benchmark.  Both move bytes: the summary
        # writes the int32 rectangle [B,H,(N-1)//32,N]; the composition reads its causal part (32c+32 entries of strip c)
        # and writes all of it.  Times are the library's per-kernel CUDA events, fractions are of the HBM copy peak.
        from dism_b200 import _lib
        peak, source = measured_peak('hbm_gbs', 6650.0)
        record = {'workload': 'strip summaries and boundary composition, labels uniform over 512 symbols', 'peak_gbs': peak,
                  'peak_source': source, 'shapes': {}}
        for b, h, n in ((8, 16, 8192), (16, 6, 2048)):
            iq, ik = [torch.randint(0, 512, (b, h, n), generator=g, device='cuda', dtype=torch.int32) for _ in range(2)]
            hard = torch.ones(b, h, dtype=torch.bool, device='cuda')
            for _ in range(args.warmup):
                cu.hard_chunk(cu.hard_summary(iq, ik, hard))
            torch.cuda.synchronize()
            _lib.load().dism_profile_enable(1)
            for _ in range(args.steps):
                cu.hard_chunk(cu.hard_summary(iq, ik, hard))
            torch.cuda.synchronize()
            times = {}
            for name, ms in _lib.kernel_timings():
                times.setdefault(name, []).append(ms)
            _lib.load().dism_profile_enable(0)
            strips = (n - 1) // 32
            rectangle = b * h * strips * n * 4
            causal = b * h * 32 * strips * (strips + 1) // 2 * 4
            moved = {'hard_summary': rectangle + 2 * b * h * n * 4, 'hard_chunk': causal + rectangle}
            record['shapes'][f'B{b} H{h} N{n}'] = {
                name: {'ms': sum(v) / len(v), 'bytes': moved[name], 'gbs': moved[name] / (sum(v) / len(v) * 1e-3) / 1e9,
                       'frac': moved[name] / (sum(v) / len(v) * 1e-3) / 1e9 / peak} for name, v in times.items()}
        record.update(steps=args.steps, warmup=args.warmup)
        print(json.dumps(record))
    else:
        batch, n = 4, 4096
        rng = np.random.default_rng(0)
        streams = np.empty((batch, n), np.int32)
        for row in range(batch):
            s = list(rng.integers(0, 256, 512))
            while len(s) < n:
                length = int(rng.integers(16, 513))
                if rng.random() < .5:
                    at = int(rng.integers(0, len(s)))
                    for t in range(length):
                        s.append(s[at + t])
                else:
                    s.extend(rng.integers(0, 256, length))
            streams[row] = s[:n]
        device = torch.from_numpy(streams).cuda()
        ms = timed(lambda: cu.longest_match(device))
        print(json.dumps({'workload': 'symbol streams [4, 4096] over 256 symbols, single longest earlier match',
                          'metric': 'positions/s', 'value': batch * n / (ms * 1e-3), 'ms': ms,
                          'steps': args.steps, 'warmup': args.warmup}))


def run_model(args):
    """The nanochat-shaped model with DISM layers (dism_b200/model.py): depth 20, width 1280, 10 heads of 128, vocabulary
    65536, bf16 weights, sequences of 2048 uniform-random tokens, batch 16 per GPU.  One step = forward, backward, the
    data-parallel gradient sum over NCCL (dism_b200/data_parallel.py) and an AdamW update; metric: tokens/s over all
    ranks, time = the slowest rank's."""
    import torch.distributed as dist
    import dism_b200
    dism_b200.install_dropin()
    from dism_b200.model import DismLM
    from dism_b200.data_parallel import sum_gradients
    rank, world = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1))
    local = int(os.environ.get('LOCAL_RANK', 0))
    torch.cuda.set_device(local)
    device = torch.device('cuda', local)
    if world > 1:
        dist.init_process_group('nccl', device_id=device)
    torch.manual_seed(0)  # the same initial weights on every rank
    depth, width, heads, head_dim, vocab, batch, seq = 20, 1280, 10, 128, 65536, args.model_batch, 2048
    model = DismLM(depth, width, heads, head_dim, vocab).to(device).bfloat16()
    optimizer = torch.optim.AdamW(model.parameters(), lr=1e-4, fused=True)
    parameters = [p for p in model.parameters()]
    generator = torch.Generator().manual_seed(1 + rank)
    host = [torch.randint(0, vocab, (batch, seq + 1), generator=generator, dtype=torch.int32).pin_memory() for _ in range(4)]

    def step(index):
        tokens = host[index % len(host)].to(device, non_blocking=True).long()
        loss = model(tokens[:, :-1], tokens[:, 1:])
        loss.backward()
        if world > 1:
            sum_gradients(parameters)
            torch._foreach_div_([p.grad for p in parameters if p.grad is not None], world)
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)
        return loss

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for index in range(args.warmup):
        step(index)
    barrier()
    with ClockSampler(local) as clocks:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for index in range(args.steps):
            loss = step(index)
        value = loss.item()  # the step's result read back on the host, inside the timed region
        stop.record()
        barrier()
    elapsed = torch.tensor([start.elapsed_time(stop)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms = float(elapsed) / args.steps
        tokens_per_second = world * batch * seq / (ms * 1e-3)
        count = sum(p.numel() for p in parameters)
        print(json.dumps({
            'metric': 'training tokens/s, nanochat-shaped model with DISM layers (fwd + bwd + gradient all-reduce + AdamW)',
            'value': tokens_per_second, 'unit': 'tokens/s', 'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': ms,
            'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic (uniform random tokens, random-init weights)',
            'config': {'workload': f'depth {depth}, width {width}, {heads} heads x {head_dim}, vocabulary {vocab}, sequence {seq}, batch {batch} per GPU',
                       'parallelism': f'dp{world}: replicas, bucketed NCCL all_reduce(SUM) of the gradients', 'parameters': count},
            'loss': value, 'per_gpu_value': tokens_per_second / world,
            'e2e': {'value': tokens_per_second, 'unit': 'tokens/s', 'h2d_bytes_per_step': batch * (seq + 1) * 4, 'd2h_bytes_per_step': 4},
            'clocks': clocks.summary()}))
    if world > 1:
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument('--gpus', type=int, default=1)
    parser.add_argument('--steps', type=int, default=10)
    parser.add_argument('--warmup', type=int, default=3)
    parser.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    # profiling aids (ncu captures want a small case and no host-side work); not for reported numbers
    parser.add_argument('--batch', type=int, default=SHAPE['batch'])
    parser.add_argument('--kernels-only', action='store_true', help='skip the end-to-end and CPU-baseline legs')
    parser.add_argument('--share', type=int, default=0, help='with --kernels-only: time the head slice one of this many GPUs would get')
    parser.add_argument('--model-batch', type=int, default=16, help='sequences per GPU of the model workload')
    parser.add_argument('--workload', default='training', choices=['training', 'long_context', 'symbol_streams', 'dense_labels', 'saved_state', 'packed', 'model'],
                        help='side workloads print their own line; the benchmark contract is the training shape')
    args = parser.parse_args()
    SHAPE['batch'] = args.batch
    if args.workload == 'model':
        run_model(args)
    elif args.workload != 'training':
        run_other_workload(args)
    elif args.impl == 'reference':
        run_reference(args)
    else:
        run_ours(args)


if __name__ == '__main__':
    main()
