"""Benchmark of the chunk-level mixed-precision optimizer step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1: the GPT-2-XL-shaped chunk set (1 557 611 200 parameters in 64 MiB fp16 chunks, fp32 master and
moments, AdamW wd 0.01, gradients ~ N(0, 1e-3) * 2^16).  One step = the single-pass step: the device-side
decision taken on the assumption of no overflow, ONE launch over all chunks that unscales, detects inf/nan,
runs AdamW out of place between two sets of master/moment arrays and writes the fp16 working copies (gradients
read from the blocks where the backward pass left them), then the device-side commit (the sets change roles, or
the update is dropped and the step becomes a skip).  ``--step probe-update`` times the two-pass form instead (one
probe launch over all gradient blocks, decision, update in place), ``--landing copy`` the older form in which
every block is first copied into its shard (fused with the probe).
N > 1 (under torchrun): the OPT-13B-shaped chunk set sharded over the ranks; one step = rank average of the
gradient blocks (reduce-scatter), decision, update of the rank's shards, all-gather of the refreshed working
copies.  ``--collective auto`` (default) runs the fastest measured form for the group size, behind a self-check
against the CPU oracle: at 2 ranks the in-place update kernel with both collectives inside over peer-mapped NVLink
memory (``p2p-fused``), from 4 ranks on ONE kernel that reduces, updates and gathers tile by tile through the
NVLink switch (``mm``); otherwise, and as fall-back, the pull reduce-scatter kernel and the update + push
all-gather kernel (``p2p``).  Also: ``p2p-overlap``, copy-engine staged (``staged``), NCCL on side streams
(``nccl``).  ``--workload opt66b_bf16``: the OPT-66B-shaped bf16 set; ``--workload residency``: one training
iteration through the wrapper under three residency modes; ``--workload probe-rate``: the inf/nan probe alone, its
load/store form against its bulk-copy ring.  ``--tune KNOB=VALUE`` sets a launch-shape knob of the library for the run
(e.g. ``adam_tma_stages=3``, ``probe_variant=0``) and is named in ``config.tuning``.

Prints ONE JSON line (rank 0).  ``value`` is whole-job parameters per second with all inputs resident
in HBM; ``roofline`` (N = 1) is the update launch against the pool-wide measured copy peak, with the DRAM traffic an
ncu capture of a small case counted (scaled; the summary under ``profiles/`` is read at run time) and the rate of a
device-to-device copy on the GPU of the run beside it; ``e2e`` is the same step through an engine method that takes pinned host buffers on both ends
(gradients in, updated low-precision parameters out: ``step_from_host`` at N = 1, ``step_sharded_p2p`` /
``step_sharded_single_pass`` with ``host_grads=`` / ``host_params=`` at N > 1); at N = 1 it is the single-pass
form (updates start while gradients still arrive and are dropped if an overflow turns up), with the plain
form's time beside it.  At N > 1 the line carries ``parity_check``: a small sharded case run through the same
engine method and compared with the CPU oracle on every rank before the warm-up.  ``--shards host`` / ``host-streamed`` (N = 1): the optimizer state kept in
pinned host memory.  ``--impl reference`` times the
reference's CPU Adam path (torch.optim.AdamW on the host cores — ColossalAI's CPUAdam is not installable
offline — next to the C oracle with all threads) on a bounded sample of the same workload.
"""
import argparse
import contextlib
import json
import os
import re
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GPT2XL_PARAMS = 48 * (12 * 1600 * 1600 + 13 * 1600) + 50257 * 1600 + 1024 * 1600 + 2 * 1600
OPT13B_PARAMS = 40 * (12 * 5120 * 5120 + 13 * 5120) + 50272 * 5120 + 2050 * 5120 + 2 * 5120
OPT66B_PARAMS = 64 * (12 * 9216 * 9216 + 13 * 9216) + 50272 * 9216 + 2050 * 9216 + 2 * 9216
CHUNK_1GPU = 32 * 1024 * 1024    # 64 MiB of fp16
CHUNK_SHARDED = 256 * 1024 * 1024    # 512 MiB of fp16
BYTES_PER_ELEM = 28    # updated element: g 2 + p/m/v 12 read, p/m/v 12 + p16 2 written
BYTES_PER_PAD_ELEM = 6    # element past valid_end: master read, working copy written


# ncu captures of the update kernel on a small case (larger than L2), summarised as text; the row that gives the DRAM
# bytes per element is read from there
TRAFFIC_PROFILES = {'single-pass': 'adam_tma_kernel_single_pass_small_case_ncu.md',
                    'probe-update': 'adam_tma_kernel_small_case_ncu.md'}


def captured_traffic_per_element(step):
    """(dram read + write bytes per element of the small-case ncu capture, the summary's file name), or (None, None)
    when the summary or its row is missing."""
    name = TRAFFIC_PROFILES.get(step)
    try:
        with open(os.path.join(ROOT, 'profiles', name)) as f:
            text = f.read()
    except (OSError, TypeError):
        return None, None
    m = re.search(r'^\|\s*traffic per element\s*\|\s*([\d ,.]+)MB\s*/\s*([\d ,]+)=', text, re.M)
    if not m:
        return None, None
    mbytes = float(m.group(1).replace(' ', '').replace(',', ''))
    elems = int(m.group(2).replace(' ', '').replace(',', ''))
    return mbytes * 1e6 / elems, name


def live_copy_gbs(device, nbytes=4 << 30, reps=5):
    """Read + write rate of a device-to-device copy of ``nbytes`` (the runtime's own copy kernel) on ``device``: the best
    of ``reps`` after two warm-up copies, CUDA events.  None if the memory for it is not there."""
    try:
        src = torch.empty(nbytes, dtype=torch.uint8, device=device)
        dst = torch.empty(nbytes, dtype=torch.uint8, device=device)
    except RuntimeError:
        return None
    src.zero_()
    best = None
    for i in range(reps + 2):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        dst.copy_(src)
        b.record()
        torch.cuda.synchronize(device)
        if i >= 2:
            ms = a.elapsed_time(b)
            best = ms if best is None else min(best, ms)
    del src, dst
    return 2 * nbytes / (best * 1e-3) / 1e9


def load_peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)['hbm_gbs']), 'measured'
    return 6650.0, 'fallback'


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 20 ms from before the warm-up;
    only samples whose timestamp falls inside the timed region are summarised."""
    QUERY = ('timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,'
             'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
             'clocks_event_reasons.sw_power_cap')

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.path = None
        self.t0 = self.t1 = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix='.csv')
            os.close(fd)
            self.proc = subprocess.Popen(['nvidia-smi', '-i', str(self.index), f'--query-gpu={self.QUERY}',
                                          '--format=csv,noheader,nounits', '-lms', '20'],
                                         stdout=open(self.path, 'w'), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def mark_begin(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    @staticmethod
    def _stamp(text):
        import datetime
        try:
            return datetime.datetime.strptime(text, '%Y/%m/%d %H:%M:%S.%f').timestamp()
        except ValueError:
            return None

    def stop(self):
        out = {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': [], 'samples': 0}
        if self.proc is None:
            return out
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        rows = []
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(',')]
                if len(parts) < 8:
                    continue
                try:
                    rows.append((self._stamp(parts[0]), float(parts[1]), float(parts[2]), float(parts[3]), parts[4:8]))
                except ValueError:
                    continue
        os.unlink(self.path)
        inside = [r for r in rows if r[0] is not None and self.t0 is not None and self.t0 <= r[0] <= self.t1]
        scope = 'timed region'
        if len(inside) < 3:
            inside, scope = rows, 'whole run (timed region shorter than the sampling period)'
        if inside:
            reasons = set()
            for r in inside:
                for name, val in zip(names, r[4]):
                    if val.lower().startswith('active'):
                        reasons.add(name)
            out.update(sm_mhz=statistics.median(r[1] for r in inside), sm_max_mhz=inside[0][2],
                       reasons=sorted(reasons), samples=len(inside), power_w_max=max(r[3] for r in inside),
                       scope=scope)
        return out


def chunk_layout(total, chunk, world):
    """(number of chunks, used elements of each chunk) when `total` parameters are packed flat."""
    n = (total + chunk - 1) // chunk
    used = [chunk] * (n - 1) + [total - chunk * (n - 1)]
    return n, used


def valid_end(used, shard, rank):
    begin = shard * rank
    return max(0, min(shard, used - begin))


def synth_master(n, device, seed):
    """Seeded fp32 master shard ~ N(0, 0.02)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    return torch.empty(n, device=device, dtype=torch.float32).normal_(0.0, 0.02, generator=gen)


def synth_grad(n, device, gen, scale, sigma, dtype, out=None):
    g = torch.empty(n, device=device, dtype=torch.float32).normal_(0.0, sigma, generator=gen).mul_(scale)
    if out is None:
        return g.to(dtype)
    out.copy_(g)
    return out


# ------------------------------------------------------------------------------------------------------
# multi-GPU parity self-check (outside the timed region)
# ------------------------------------------------------------------------------------------------------


_KEEP_ALIVE = []


def sharded_parity_check(collective, world, rank, device, group, seed):
    """Run a small sharded case through the SAME engine method the benchmark times and compare it, on every
    rank, with the CPU oracle (used here only as the checker): ragged chunks, a chunk whose used length ends
    inside one rank's shard, a chunk that fits in the first shard, one inf that lands in rank 0's shard only
    (every rank must skip), five steps, fp16 and bf16.  Checked: the reduced gradients bit for bit (NVLink
    paths) or to fp16 rounding (NCCL, whose summation order is its own), skip decision, loss scale and step
    count on all ranks, fp32 masters within 1e-6 of the double-precision oracle, and the gathered block equal
    to all ranks' refreshed shards.  Returns (ok, number of cases, first failure or None), agreed across ranks."""
    import torch.distributed as dist
    from elixir_b200 import comm
    from elixir_b200 import kernels as K
    from elixir_b200.engine import ChunkStepEngine
    from elixir_b200.scaler import DynamicGradScaler
    from oracle import oracle as orc

    def bits_equal(a, b):
        a, b = a.detach().cpu().contiguous(), b.detach().cpu().contiguous()
        view = {2: torch.int16, 4: torch.int32}[a.element_size()]
        return a.shape == b.shape and a.dtype == b.dtype and torch.equal(a.view(view), b.view(view))

    def close(actual, ref64, rtol=2e-6):
        a, r = actual.detach().double().cpu(), ref64.double()
        bound = rtol * torch.maximum(r.abs(), r.pow(2).mean().sqrt().expand_as(r)).clamp(min=1e-45)
        return bool(((a - r).abs() <= bound).all())

    failure, cases = None, 0
    for dtype in (torch.float16, torch.bfloat16):
        cases += 1
        scale = 256.0
        chunk_sizes = [world * 4096 * 40, world * (4096 + 16), world * 4096 * 5, world * 24]
        used = [chunk_sizes[0], chunk_sizes[1], chunk_sizes[2] // 2 + 7, 9]
        engine = ChunkStepEngine(device, dtype, DynamicGradScaler(initial_scale=scale, hysteresis=1, growth_interval=3),
                                 process_group=group)
        # switch-side sum: the oracle steps on the averaged gradients as fp32 values (float(sum) / W, what the kernel feeds
        # to Adam); otherwise on the reduced low-precision shard
        host_dtype = torch.float32 if collective == 'mm' else dtype
        host, host_ctl, host_state = orc.ChunkSet(host_dtype), orc.new_ctl(scale), []
        hypers = [K.hyper(weight_decay=0.01)]
        for c, (C, u) in enumerate(zip(chunk_sizes, used)):
            S = C // world
            gen = torch.Generator().manual_seed(seed + c)
            full = torch.randn(C, generator=gen) * 0.02
            full[u:] = 0
            mine = full[rank * S:(rank + 1) * S].clone()
            nv = max(0, min(S, u - rank * S))
            lowp = torch.zeros(S, dtype=host_dtype)
            host.add_chunk(mine, torch.zeros(S), torch.zeros(S), lowp, nv, [(0, nv, 0)] if nv else [])
            host_state.append((mine, lowp))
            engine.add_shard(mine.to(device), torch.zeros(S, dtype=dtype, device=device), nv, [(0, nv, 0)] if nv else [])
        engine.finalize()
        engine.set_hyper(hypers)
        if collective == 'mm':
            engine.enable_single_pass()
            engine.enable_multicast(chunk_sizes, timeout_ms=5000)
            gather = [engine.gather_block(c) for c in range(len(chunk_sizes))]
        elif collective in ('p2p', 'p2p-fused', 'p2p-overlap', 'staged'):
            engine.enable_p2p(chunk_sizes, timeout_ms=5000)
            if collective == 'staged':
                engine.enable_staging(pool=2)
            gather = [engine.gather_block(c) for c in range(len(chunk_sizes))]
        else:
            gather = [torch.empty(C, dtype=dtype, device=device) for C in chunk_sizes]
        for step in range(5):
            per_rank, blocks = [], []
            for c, C in enumerate(chunk_sizes):
                rank_grads = []
                for r in range(world):
                    gen = torch.Generator().manual_seed(seed + 1000 * step + 10 * c + r)
                    g = (torch.randn(C, generator=gen) * 1e-3 * host_ctl.scale).to(dtype)
                    if step == 2 and c == 1 and r == world - 1:
                        g[5] = float('inf')    # lands in rank 0's shard only
                    rank_grads.append(g)
                per_rank.append(rank_grads)
                if collective in ('p2p', 'p2p-fused', 'p2p-overlap', 'staged', 'mm'):
                    engine.grad_block(c).copy_(rank_grads[rank])
                else:
                    blocks.append(rank_grads[rank].to(device))
            reduced = []
            if collective == 'mm':
                # the switch's sum has an arithmetic of its own, as NCCL's order is its own: parity of the step is defined
                # GIVEN the reduced gradients, captured here with the same switch operation before the step consumes them
                torch.cuda.synchronize()
                dist.barrier(group=group)
                sums = [t.cpu() for t in engine.switch_reduced_gradients()]
                torch.cuda.synchronize()
                dist.barrier(group=group)
            for c, C in enumerate(chunk_sizes):
                S = C // world
                mine = [g[rank * S:(rank + 1) * S].contiguous() for g in per_rank[c]]
                if collective == 'mm':
                    exact = torch.stack([m.double() for m in mine]).sum(0)
                    finite = torch.isfinite(exact)
                    ulp = 2.0**-10 if dtype == torch.float16 else 2.0**-7
                    bound = world * ulp * torch.stack([m.double().abs() for m in mine]).sum(0)
                    if not torch.equal(torch.isfinite(sums[c].double()), finite) or \
                            not bool(((sums[c].double() - exact).abs()[finite] <= bound[finite]).all()):
                        failure = failure or f'{dtype} step {step} chunk {c}: switch-side sum off the exact sum by more than its roundings'
                    reduced.append(sums[c].float() * (1.0 / world))
                elif collective in ('p2p', 'p2p-fused', 'p2p-overlap', 'staged'):
                    reduced.append(orc.reduce_avg_f32acc(mine))    # rank-order fp32 accumulation, one rounding
                else:
                    out = torch.empty(S, dtype=dtype, device=device)
                    comm.reduce_scatter_avg(out, blocks[c].clone(), group)
                    reduced.append(out.cpu())
                    want = orc.reduce_avg(mine).float()
                    finite = torch.isfinite(want)
                    if not torch.equal(finite, torch.isfinite(reduced[c].float())) or float(
                            (reduced[c].float() - want).abs()[finite].max()) > 2 * 2.0**-8 * float(want.abs()[finite].max()):
                        failure = failure or f'{dtype} step {step} chunk {c}: NCCL average off the divide-then-sum value'
            if collective == 'p2p':
                engine.step_sharded_p2p()
            elif collective == 'p2p-overlap':
                engine.step_sharded_probe_first(pull_ctas=40)
            elif collective == 'p2p-fused':
                engine.step_sharded_pull_push()
            elif collective == 'mm':
                engine.step_sharded_single_pass()
            elif collective == 'staged':
                engine.step_sharded_staged()
            else:
                engine.step_sharded(blocks, gather)
            torch.cuda.synchronize()
            shards = engine.current_shards()
            for c in range(len(chunk_sizes)):
                host_state[c][1].copy_(reduced[c])
            if step == 2:
                host_ctl.found_inf = 1    # agreement: every rank skips, also those whose shards are clean
            skipped = host.step(host_ctl, engine.scaler.cfg, hypers, probe=True, f64=True)
            ctl = engine.read_control()
            if ctl.status or bool(ctl.skip) != skipped or skipped != (step == 2) or \
                    (ctl.scale, ctl.step) != (host_ctl.scale, host_ctl.step):
                failure = failure or f'{dtype} step {step}: control block status={ctl.status} skip={ctl.skip} scale={ctl.scale}'
            for c, C in enumerate(chunk_sizes):
                S = C // world
                if not close(shards[c][0], host_state[c][0]):
                    failure = failure or f'{dtype} step {step} chunk {c}: master off the oracle'
                want16 = torch.empty(S, dtype=dtype)
                orc.cast(shards[c][0].cpu(), want16)
                if not bits_equal(shards[c][3], want16):
                    failure = failure or f'{dtype} step {step} chunk {c}: working copy is not the rounded master'
                others = [torch.empty_like(shards[c][3]) for _ in range(world)]
                dist.all_gather(others, shards[c][3], group=group)
                if not bits_equal(gather[c], torch.cat(others)):
                    failure = failure or f'{dtype} step {step} chunk {c}: gathered block differs from the ranks\' shards'
        _KEEP_ALIVE.append(engine)    # peer-mapped buffers stay allocated while other ranks have them mapped
    verdict = torch.tensor([0 if failure is None else 1], device=device)
    dist.all_reduce(verdict, op=dist.ReduceOp.MAX, group=group)
    return verdict.item() == 0, cases, failure


# ------------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------------


def run_ours(args):
    import torch.distributed as dist
    from elixir_b200 import kernels as K
    from elixir_b200.engine import ChunkStepEngine
    from elixir_b200.scaler import DynamicGradScaler

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    if world != args.gpus:
        raise SystemExit(f'--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run')
    torch.cuda.set_device(local_rank)
    device = torch.device('cuda', local_rank)
    group = None
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        dist.init_process_group('nccl', rank=rank, world_size=world, device_id=device)
        group = dist.group.WORLD

    parity = None
    if world > 1 and not args.no_parity_check:
        what = ('small ragged chunk set, 5 steps (1 skipped by an inf in one rank\'s shard), fp16 and bf16, against the CPU '
                'oracle on every rank')
        note = None
        preferred = args.collective_was_auto and args.collective != 'p2p'
        if preferred:
            # the variant --collective auto prefers at this size has requirements of its own (the switch-side path:
            # multicast support of GPUs, driver and torch): where its self-check does not come out clean the
            # benchmark falls back to the two peer-mapped kernels instead of giving up
            try:
                ok, cases, failure = sharded_parity_check(args.collective, world, rank, device, group, args.seed)
            except Exception as exc:    # noqa: BLE001
                ok, cases, failure = False, 0, f'{type(exc).__name__}: {exc}'
            agreed = torch.tensor([1 if ok else 0], device=device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
            if not agreed.item():
                note = f'--collective auto: {args.collective} did not pass its self-check here ({failure}); using p2p'
                if rank == 0:
                    print('bench: ' + note, file=sys.stderr)
                args.collective = 'p2p'
        if note is not None or not preferred:
            ok, cases, failure = sharded_parity_check(args.collective, world, rank, device, group, args.seed)
        parity = {'ok': ok, 'world': world, 'cases': cases, 'collective': args.collective, 'what': what}
        if note:
            parity['note'] = note
        if not ok:
            if failure:
                print(f'bench: parity check failed on rank {rank}: {failure}', file=sys.stderr)
            dist.barrier()
            dist.destroy_process_group()
            raise SystemExit(3)

    dtype, sigma = torch.float16, 1e-3
    if world == 1:
        workload, total, chunk, scale, wd = 'gpt2xl_chunks_1gpu', GPT2XL_PARAMS, CHUNK_1GPU, 65536.0, 0.01
    elif args.workload == 'opt66b_bf16':
        # OPT-66B-shaped set: bf16 chunks, constant scale 1, AdamW, ~8.2 G elements of state per rank at W = 8.
        # The replicated blocks cannot all be resident next to 115 GB of state, so they come from a small pool,
        # as in training, and the step runs chunk by chunk.
        workload, total, chunk, scale, wd = f'opt66b_bf16_chunks_sharded_w{world}', OPT66B_PARAMS, CHUNK_SHARDED, 1.0, 0.01
        dtype, sigma = torch.bfloat16, 1e-4
        args.pool = args.pool or 4
    else:
        workload, total, chunk, scale, wd = f'opt13b_chunks_sharded_w{world}', OPT13B_PARAMS, CHUNK_SHARDED, 1024.0, 0.0
    if args.shards != 'device':
        if world != 1:
            raise SystemExit('--shards host is a 1-GPU measurement (the collectives write device-resident shards)')
        workload, args.no_e2e = workload + '_' + args.shards.replace('-', '_') + '_shards', True
    if args.params:
        total, workload = args.params, workload + f'_params{args.params}'
    if args.chunk_elems:
        chunk, workload = args.chunk_elems, workload + f'_chunk{args.chunk_elems}'
    n_chunks, used = chunk_layout(total, chunk, world)
    shard = chunk // world
    if world > 1 and args.collective == 'mm':
        # two sets of master and moments (26 B per element with the working copy) next to the two slabs of
        # replicated blocks: refuse cleanly, before anything is allocated, where that does not fit
        need = n_chunks * shard * 26 + 2 * n_chunks * chunk * 2
        free, _ = torch.cuda.mem_get_info(device)
        if need > 0.95 * free and args.collective_was_auto:
            args.collective = 'p2p'    # (the self-check above ran on the switch-side path; the timed step is p2p)
        elif need > 0.95 * free:
            raise SystemExit(f'bench: --collective mm needs {need / 1e9:.0f} GB per GPU at {world} ranks for this workload '
                             f'({free / 1e9:.0f} GB free); use --collective p2p')

    if dtype == torch.bfloat16:
        from elixir_b200.scaler import ConstantGradScaler
        scaler = ConstantGradScaler(1.0)
    else:
        scaler = DynamicGradScaler(initial_scale=scale, growth_factor=2, backoff_factor=0.5, growth_interval=1000,
                                   min_scale=1, max_scale=2**24, hysteresis=2)
    engine = ChunkStepEngine(device, dtype, scaler, process_group=group)
    in_place_sources = world == 1 and args.shards == 'device' and args.landing == 'none'
    grad_blocks, n_valid_total = [], 0
    for c in range(n_chunks):
        master = synth_master(shard, device, args.seed + 1000 * rank + c)
        nv = valid_end(used[c], shard, rank)
        if nv < shard:
            master[nv:].zero_()
        lowp = torch.empty(shard, dtype=dtype, device=device)
        K.cast_copyback(master, lowp)
        if args.shards != 'device':
            # the reference's shard_device=cpu placement: master, moments and working copy in pinned host
            # memory, updated in place over PCIe by the same kernels
            master, lowp = master.cpu().pin_memory(), lowp.cpu().pin_memory()
        src = None
        if in_place_sources:
            # the gradient block of this chunk: the probe and the update read it where it is
            gen = torch.Generator(device=device).manual_seed(args.seed + 7919 * (c + 1))
            src = synth_grad(shard, device, gen, scale, sigma, dtype)
            grad_blocks.append(src)
        engine.add_shard(master, lowp, nv, [(0, nv, 0)] if nv else [], grad_src=src)
        n_valid_total += nv
    engine.finalize()
    engine.set_hyper([K.hyper(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=wd, adamw_mode=True)])
    if args.shards == 'host-streamed':
        engine.enable_streaming(slots=3)
    single_pass = in_place_sources and args.step == 'single-pass'
    if single_pass or (world > 1 and args.collective == 'mm'):
        engine.enable_single_pass()    # second set of master and moments: the update runs out of place

    # gradient sources
    if world == 1:
        if not in_place_sources:
            for c in range(n_chunks):
                gen = torch.Generator(device=device).manual_seed(args.seed + 7919 * (c + 1))
                grad_blocks.append(synth_grad(shard, device, gen, scale, sigma, dtype))
        gather_blocks = None
    elif args.collective in ('p2p', 'p2p-fused', 'p2p-overlap', 'staged', 'mm'):
        # NVLink path: every chunk owns a block in the peer-mapped gradient and gather slabs
        if args.collective == 'mm':
            engine.enable_multicast([chunk] * n_chunks)
        else:
            engine.enable_p2p([chunk] * n_chunks, pool=(args.pool or None) if args.collective == 'p2p' else None)
        if args.collective == 'staged':
            engine.enable_staging(pool=4)
        seeds = 4
        for c in range(min(n_chunks, args.pool) if args.pool else n_chunks):
            if c < seeds:
                gen = torch.Generator(device=device).manual_seed(args.seed + 7919 * (c + 1) + 31 * rank)
                synth_grad(chunk, device, gen, scale, sigma, dtype, out=engine.grad_block(c))
            else:
                engine.grad_block(c).copy_(engine.grad_block(c % seeds))
        grad_blocks = [engine.grad_block(c) for c in range(n_chunks)]
        gather_blocks = [engine.gather_block(c) for c in range(n_chunks)]
    else:
        pool = 4
        grad_pool, gather_pool = [], []
        for b in range(pool):
            gen = torch.Generator(device=device).manual_seed(args.seed + 7919 * (b + 1) + 31 * rank)
            grad_pool.append(synth_grad(chunk, device, gen, scale, sigma, dtype))
            gather_pool.append(torch.empty(chunk, dtype=dtype, device=device))
        grad_blocks = [grad_pool[c % pool] for c in range(n_chunks)]
        gather_blocks = [gather_pool[c % pool] for c in range(n_chunks)]

    adam_events = []

    def one_step(record=False):
        if world == 1 and args.shards == 'host-streamed':
            engine.land_all(grad_blocks, streams=args.land_streams)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            engine.step_streamed()    # decision, then copy in / update / copy out per chunk on three streams
            b.record()
            if record:
                adam_events.append((a, b))
        elif single_pass:
            # ChunkStepEngine.step_single_pass, spelled out so that the update launch can be timed on its own
            (t0, _), (t1, _) = engine._sets
            K.step_begin_optimistic(engine.ctl, engine.scaler.cfg, engine.chunk_flags)
            if record:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
            K.adam_multi_single_pass(t0, t1, engine.ctl, engine.chunk_flags)
            if record:
                b.record()
                adam_events.append((a, b))
            K.step_commit(engine.ctl, engine.scaler.cfg, engine.chunk_flags)
            K.adam_multi_repair(t0, t1, engine.ctl)
        elif world == 1:
            if in_place_sources:
                engine.probe()
            else:
                engine.land_all(grad_blocks, streams=args.land_streams)
            engine.begin_step()
            if record:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                engine.update()
                b.record()
                adam_events.append((a, b))
            else:
                engine.update()
            engine.end_step()
        elif args.collective == 'p2p':
            engine.step_sharded_p2p()
        elif args.collective == 'p2p-overlap':
            engine.step_sharded_probe_first(pull_ctas=args.pull_ctas)
        elif args.collective == 'p2p-fused':
            engine.step_sharded_pull_push()
        elif args.collective == 'mm':
            engine.step_sharded_single_pass()
        elif args.collective == 'staged':
            engine.step_sharded_staged()
        else:
            engine.step_sharded(grad_blocks, gather_blocks)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        barrier()
        ms = a.elapsed_time(b)
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        return ms

    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(args.warmup):
        one_step()
    torch.cuda.synchronize()
    sampler.mark_begin()
    total_ms = timed(lambda: one_step(record=True), args.steps)
    sampler.mark_end()
    clocks = sampler.stop()
    ms_per_step = total_ms / args.steps
    ctl = engine.read_control()
    if ctl.status or ctl.skipped_steps:
        raise SystemExit(f'bench: unexpected control state status={ctl.status} skipped={ctl.skipped_steps}')

    peak, peak_kind = load_peaks()
    result = {
        'metric': 'chunk Adam Gparams/s',
        'value': total / (ms_per_step * 1e-3) / 1e9,
        'unit': 'Gparams/s',
        'n_gpus': world,
        'steps': args.steps,
        'warmup': args.warmup,
        'ms_per_step': ms_per_step,
        'higher_is_better': True,
        'scaling': 'weak' if world == 1 else 'strong',
        'vs_baseline': None,
        'dtype': 'f32',
        'data': 'synthetic',
        'config': {
            'workload': workload,
            **({'tuning': list(args.tune)} if args.tune else {}),
            'params': total,
            'chunk_elems': chunk,
            'n_chunks': n_chunks,
            'grad_dtype': 'bf16' if dtype == torch.bfloat16 else 'fp16',
            'optimizer': f'AdamW lr1e-3 b(0.9,0.999) eps1e-8 wd{wd}',
            'loss_scale': scale,
            'l2_policy': 'inputs larger than L2 (state per GPU %.1f GB)' % (
                engine.n_elements() * (26 if engine._sets is not None else 14) / 1e9),
            'layout': 'flat packing, tensors may straddle chunks',
            'block_pool': args.pool or n_chunks,
            'collectives': 'none (1 GPU)' if world == 1 else
                           ('fused into the kernels over peer-mapped NVLink memory (pull reduce-scatter + probe, '
                            'Adam + push all-gather)' if args.collective == 'p2p' else
                            'both collectives inside the in-place update kernel over peer-mapped NVLink memory (per tile: bulk loads '
                            'of every rank\'s gradient slice, rank average, Adam, bulk stores to every rank\'s gather block); '
                            'the overflow decision is taken first, from a probe of every rank\'s own gradient blocks'
                            if args.collective == 'p2p-fused' else
                            'the same two kernels chunk by chunk on two streams, the update of a chunk running while the next '
                            'one is reduced; the overflow decision is taken first, from a probe of every rank\'s own gradient '
                            'blocks' if args.collective == 'p2p-overlap' else
                            'ONE kernel per step through the NVLink switch: per tile the sum of all ranks\' gradients '
                            '(multimem.ld_reduce), Adam out of place with inf/nan detection, working copy to all ranks '
                            '(multimem.st); symmetric memory' if args.collective == 'mm' else
                            'copy engines over peer-mapped NVLink memory (staged reduce + probe kernel, fused update, '
                            'copies into the gather blocks)' if args.collective == 'staged' else
                            'NCCL reduce-scatter (pre-multiplied sum) and all-gather per chunk on side streams'),
        },
        'clocks': clocks,
        'context': {'reference_planner_gpu_adam_gparams_per_s_per_gpu': 50.0,
                    'note': 'constant fitted by the reference authors on unnamed hardware for fp32 gradients without the '
                            'copy-back (elixir/search/simulator.py:128-129); not this exact metric, hence vs_baseline null'},
    }

    if world == 1:
        adam_ms = statistics.mean(a.elapsed_time(b) for a, b in adam_events)
        n_elems = engine.n_elements()
        # algorithmic bytes of one update launch: 28 per updated element, 6 per element past valid_end
        algo_bytes = BYTES_PER_ELEM * n_valid_total + BYTES_PER_PAD_ELEM * (n_elems - n_valid_total)
        achieved = algo_bytes / (adam_ms * 1e-3) / 1e9
        # DRAM traffic of one launch: counted by ncu on a small case of the same kernel (the full-size launch is not
        # captured), scaled by the algorithmic bytes, which is what the traffic is proportional to
        per_elem, traffic_source = captured_traffic_per_element(args.step)
        if args.ncu_traffic_bytes:
            traffic, traffic_source = args.ncu_traffic_bytes, 'command line (--ncu-traffic-bytes)'
        elif per_elem is not None and args.shards == 'device' and args.landing == 'none':
            traffic = per_elem / BYTES_PER_ELEM * algo_bytes
            traffic_source = (f'profiles/{traffic_source}: {per_elem:.2f} B per element on the captured small case, '
                              'scaled to this launch by its algorithmic bytes')
        else:
            traffic, traffic_source = None, None
        result['roofline'] = {
            'bound': 'hbm', 'kernel': 'adam_tma_kernel', 'achieved': achieved, 'peak': peak, 'unit': 'GB/s',
            'frac': achieved / peak, 'peak_kind': peak_kind, 'ms_per_launch': adam_ms,
            'elements_per_launch': n_elems, 'updated_elements_per_launch': n_valid_total,
            'algorithmic_bytes_per_launch': algo_bytes,
            'bytes_per_element': {'updated': BYTES_PER_ELEM, 'past_valid_end': BYTES_PER_PAD_ELEM},
            'traffic': traffic, 'traffic_source': traffic_source,
            'frac_of_8TBs_nominal': achieved / 8000.0,
        }
        result['adam_gparams_per_s'] = n_elems / (adam_ms * 1e-3) / 1e9
        # the GPUs of the pool differ by several per cent: a device-to-device copy timed on THIS one, after the timed
        # region, beside the pool-wide peak the fraction above refers to
        live = live_copy_gbs(device)
        result['roofline']['this_gpu_copy_gbs'] = live
        result['roofline']['frac_of_this_gpu_copy'] = achieved / live if live else None
        if args.shards != 'device':
            per_dir = n_elems * (BYTES_PER_ELEM // 2) / (adam_ms * 1e-3) / 1e9
            result['roofline'] = {
                'bound': 'pcie',
                'kernel': ('adam_kernel (load/store variant) on pinned host shards' if args.shards == 'host' else
                           'copy engines in and out of three staging sets around adam_tma_kernel'),
                'achieved': per_dir, 'peak': 64.0, 'unit': 'GB/s per direction', 'frac': per_dir / 64.0,
                'peak_kind': 'nominal PCIe Gen5 x16 (no measured figure on this pool)', 'ms_per_launch': adam_ms,
                'elements_per_launch': n_elems, 'bytes_per_element_each_direction': BYTES_PER_ELEM // 2, 'traffic': None,
            }
        result['gpu_launches'] = args.steps * (4 if single_pass else (1 if in_place_sources else n_chunks) + 2)
        result['config']['step'] = ('single pass: inf/nan detection inside the update kernel, out of place between two state sets'
                                    if single_pass else 'probe launch(es), decision, update launch')
    else:
        bus_bytes = 2 * chunk * (world - 1) / world * n_chunks    # per collective kind, per rank, per step
        nominal, peer_copy = 900.0, 770.0    # GB/s per direction: NVLink 5 nominal; one copy-engine peer copy on this pool
        result['collective'] = {
            'per_step_bus_bytes_rs': bus_bytes, 'per_step_bus_bytes_ag': bus_bytes,
            'combined_bus_gbs': 2 * bus_bytes / (ms_per_step * 1e-3) / 1e9,
            'nominal_gbs_per_direction': nominal, 'peer_copy_gbs_per_direction': peer_copy,
        }
        # update/push phase: the 28 B/element of the update + 2 B/element for this rank's slot of its own gather block
        adam_bytes = engine.n_elements() * (BYTES_PER_ELEM + 2)
        # the step is two phases in sequence, each bounded by the slower of its NVLink and its HBM time:
        # pull reduce-scatter (NVLink; HBM only reads and writes the own slice) and update + push all-gather
        link_ms = bus_bytes / (nominal * 1e9) * 1e3
        adam_hbm_ms = adam_bytes / (peak * 1e9) * 1e3
        pull_hbm_ms = engine.n_elements() * 2 * 2 / (peak * 1e9) * 1e3
        target_ms = max(link_ms, pull_hbm_ms) + max(link_ms, adam_hbm_ms)
        achieved = 2 * bus_bytes / (ms_per_step * 1e-3) / 1e9
        result['roofline'] = {
            'bound': 'nvlink', 'achieved': achieved, 'peak': nominal, 'unit': 'GB/s', 'frac': achieved / nominal,
            'peak_kind': 'nominal NVLink 5 rate per direction', 'frac_of_peer_copy_rate': achieved / peer_copy,
            'traffic': None, 'adam_hbm_ms_at_peak': adam_hbm_ms, 'link_ms_per_collective_at_peak': link_ms,
            'target_ms': target_ms, 'frac_of_target': target_ms / ms_per_step,
            'target_note': 'max(NVLink at 900 GB/s, HBM) time of the pull phase + max(NVLink, HBM) time of the update/push phase',
        }
        if args.collective == 'mm':
            # one kernel carries both collectives and the update: its bound is the slower of the links (each direction
            # carries the switch-side sum in and the shard out once, plus every rank's share of the other transfers:
            # (W + 1) / W of the chunk bytes) and HBM (per own element: master and moments in and out 24 B, working copy
            # 2 B, plus what the switch reads from this rank's gradient blocks, 2 W B, and writes into its gather
            # blocks, 2 W B; the reduced gradient itself never touches memory)
            wire = 2 * chunk * (world + 1) / world * n_chunks
            mm_link_ms = wire / (nominal * 1e9) * 1e3
            mm_hbm_ms = engine.n_elements() * (26 + 4 * world) / (peak * 1e9) * 1e3
            result['roofline'].update(
                wire_bytes_per_direction=wire, wire_gbs_per_direction=wire / (ms_per_step * 1e-3) / 1e9,
                target_ms=max(mm_link_ms, mm_hbm_ms), frac_of_target=max(mm_link_ms, mm_hbm_ms) / ms_per_step,
                target_note='one kernel: max(NVLink time of (W + 1) / W of the chunk bytes per direction at 900 GB/s, HBM time)',
                note='achieved / frac keep the reduce-scatter + all-gather bus-byte convention (2 (W - 1) / W of the chunk '
                     'bytes per collective) so that the variants compare; the switch-side sum moves fewer bytes than that')
            result['gpu_launches'] = args.steps * 7
            result['phases_ms'] = mm_phases(engine)
        elif args.collective == 'p2p-fused':
            # one kernel behind the probe of the inputs: bounded by the slower of the links (both collectives share
            # them) and HBM (own gradient slice 2 B, master and moments 24 B, working copy 2 B, own gather slot 2 B
            # per own element, plus what the peers read from this rank's blocks and write into its gather blocks)
            probe_ms = n_chunks * chunk * 2 / (peak * 1e9) * 1e3
            hbm_ms = engine.n_elements() * (30 + 4 * (world - 1)) / (peak * 1e9) * 1e3
            result['roofline'].update(
                target_ms=probe_ms + max(2 * link_ms, hbm_ms), frac_of_target=(probe_ms + max(2 * link_ms, hbm_ms)) / ms_per_step,
                target_note='probe of the own gradient blocks at the HBM rate + one kernel: max(NVLink time of both collectives '
                            'at 900 GB/s, HBM time)')
            result['gpu_launches'] = args.steps * 7
            result['phases_ms'] = fused_phases(engine)
        elif args.collective == 'p2p-overlap':
            # one pipelined phase behind the probe of the inputs: bounded by the slower of the links (both collectives
            # share them) and HBM (probe of the own blocks 2 B x C, pull 4 B and update + push 30 B per own element)
            probe_ms = n_chunks * chunk * 2 / (peak * 1e9) * 1e3
            hbm_ms = engine.n_elements() * (4 + BYTES_PER_ELEM + 2) / (peak * 1e9) * 1e3
            result['roofline'].update(
                target_ms=probe_ms + max(2 * link_ms, hbm_ms), frac_of_target=(probe_ms + max(2 * link_ms, hbm_ms)) / ms_per_step,
                target_note='probe of the own gradient blocks at the HBM rate + max(NVLink time of both collectives at 900 GB/s, '
                            'HBM time of pull + update + push)')
            result['gpu_launches'] = args.steps * (2 * n_chunks + 5)
        elif args.collective == 'p2p' and args.pool:
            result['gpu_launches'] = args.steps * (3 * n_chunks + 3)
        elif args.collective == 'p2p':
            result['gpu_launches'] = args.steps * 6
            result['phases_ms'] = p2p_phases(engine)
        elif args.collective == 'staged':
            result['gpu_launches'] = args.steps * (2 * n_chunks + 4)
            engine.profile = True
            one_step()
            torch.cuda.synchronize()
            result['phases_ms'] = engine.phase_ms()
            engine.profile = False
        else:
            result['gpu_launches'] = args.steps * (2 * n_chunks + 1)
            # one more, untimed, step with phase timestamps: where the step time goes
            engine.profile = True
            one_step()
            torch.cuda.synchronize()
            result['phases_ms'] = engine.phase_ms()
            engine.profile = False

    # ---- end to end: pinned host buffers on both ends --------------------------------------------
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(args, engine, world, rank, device, dtype, n_chunks, shard, chunk, scale, sigma, total, timed,
                      grad_blocks, gather_blocks)
    result['e2e'] = e2e
    if parity is not None:
        result['parity_check'] = parity
    engine.check_status()

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        result['cpu_baseline'] = cpu_baseline(args, chunk, scale, sigma, wd, steps=3, chunks=4)
    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def mm_phases(engine):
    """CUDA-event time of the one fused kernel of an (untimed) single-pass sharded step, barriers not included."""
    from elixir_b200 import kernels as K
    (t0, _), (t1, _) = engine._sets
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    engine.peer_barrier(engine.ctl)
    K.step_begin_optimistic(engine.ctl, engine.scaler.cfg, engine.chunk_flags)
    ev[0].record()
    K.adam_multi_single_pass(t0, t1, engine.ctl, engine.chunk_flags, grads_table=engine.grad_slab.table,
                             gather_table=engine.gather_slab.table, block_off=engine.block_off,
                             grads_mc=engine.grad_slab.mc_ptr, gather_mc=engine.gather_slab.mc_ptr)
    ev[1].record()
    engine.peer_barrier(engine.ctl, exchange_overflow=True)
    K.step_commit(engine.ctl, engine.scaler.cfg, engine.chunk_flags)
    K.adam_multi_repair(t0, t1, engine.ctl, gather_table=engine.gather_slab.table, block_off=engine.block_off)
    engine.peer_barrier(engine.ctl)
    torch.cuda.synchronize()
    return {'reduce_adam_gather_one_kernel': ev[0].elapsed_time(ev[1])}


def fused_phases(engine):
    """CUDA-event times of the probe of the inputs and of the one fused kernel of an (untimed) p2p-fused step."""
    from elixir_b200 import kernels as K
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    engine.peer_barrier(engine.ctl)
    ev[0].record()
    K.grad_check(engine.grad_slab.local, ctl=engine.ctl)
    ev[1].record()
    engine.peer_barrier(engine.ctl, exchange_overflow=True)
    K.step_begin(engine.ctl, engine.scaler.cfg, None, engine.chunk_flags)
    ev[2].record()
    K.adam_multi_pull_push(engine.table, engine.ctl, engine.grad_slab.table, engine.gather_slab.table, engine.block_off)
    ev[3].record()
    engine.peer_barrier(engine.ctl)
    torch.cuda.synchronize()
    return {'probe_of_own_gradient_blocks': ev[0].elapsed_time(ev[1]), 'reduce_adam_gather_one_kernel': ev[2].elapsed_time(ev[3])}


def p2p_phases(engine):
    """CUDA-event time of the two fused kernels of one (untimed) NVLink step, barriers included in neither."""
    from elixir_b200 import kernels as K
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    engine.peer_barrier(engine.ctl)
    ev[0].record()
    K.pull_reduce_multi(engine.table, engine.grad_slab.table, engine.block_off, engine.ctl, chunk_flags=engine.chunk_flags)
    ev[1].record()
    engine.peer_barrier(engine.ctl, exchange_overflow=True)
    K.step_begin(engine.ctl, engine.scaler.cfg)
    ev[2].record()
    K.adam_multi_push(engine.table, engine.ctl, engine.gather_slab.table, engine.block_off)
    ev[3].record()
    engine.end_step()
    engine.peer_barrier(engine.ctl)
    torch.cuda.synchronize()
    return {'pull_reduce_probe': ev[0].elapsed_time(ev[1]), 'adam_push_gather': ev[2].elapsed_time(ev[3])}


def run_e2e(args, engine, world, rank, device, dtype, n_chunks, shard, chunk, scale, sigma, total, timed,
            grad_blocks=None, gather_blocks=None):
    """The same step with pinned host buffers on both ends, H2D and D2H inside the timed region.
    1 GPU: reduced fp16 gradients of every shard come from the host, updated fp16 parameters go back.
    Sharded: every rank's replicated gradient blocks come from the host before their reduce-scatter and
    every rank's updated shard goes back after the update (the all-gather still runs on the device)."""
    pool = min(n_chunks, 8 if world == 1 else 4)
    in_elems = shard if world == 1 else chunk
    from elixir_b200.numa import near_gpu
    host_in, host_out = [], []
    for b in range(pool):
        gen = torch.Generator().manual_seed(args.seed + 104729 * (b + 1) + rank)
        g = torch.empty(in_elems, dtype=torch.float32).normal_(0.0, sigma, generator=gen).mul_(scale).to(dtype)
        # pinned buffers on the GPU's own NUMA node where this process may run there (--no-numa: wherever it runs)
        with (contextlib.nullcontext(set()) if args.no_numa else near_gpu(device)) as numa_cpus:
            host_in.append(g.pin_memory())
            host_out.append(torch.empty(shard, dtype=dtype).pin_memory())
    grads = [host_in[c % pool] for c in range(n_chunks)]
    outs = [host_out[c % pool] for c in range(n_chunks)]
    conservative_ms = None
    engine.normalize_sets()    # after single-pass steps: the in-place legs below work on the live state set
    if world == 1:
        # first the step that waits for the last gradient before it updates anything, then the speculative one
        # (updates into a second set of master/moment arrays while gradients still arrive; adopted unless an
        # overflow turns up): same results, PCIe busy in both directions at once
        plain = lambda: engine.step_from_host(grads, outs)    # noqa: E731
        if args.no_speculation:
            fn = plain
        else:
            for _ in range(2):
                plain()
            conservative_ms = timed(plain, max(1, min(args.steps, args.e2e_steps))) / max(1, min(args.steps, args.e2e_steps))
            engine.enable_speculation()
            fn = lambda: engine.step_from_host(grads, outs, speculative=True)    # noqa: E731
    elif args.collective in ('p2p', 'p2p-fused', 'p2p-overlap'):
        # chunk by chunk: block k filled from the host while earlier chunks are pulled, shard k copied out behind
        # its update while later chunks are updated and pushed
        fn = lambda: engine.step_sharded_p2p(host_grads=grads, host_params=outs)    # noqa: E731
    elif args.collective == 'mm':
        fn = lambda: engine.step_sharded_single_pass(host_grads=grads, host_params=outs)    # noqa: E731
    elif args.collective == 'staged':
        def fn():
            for k in range(n_chunks):
                grad_blocks[k].copy_(grads[k], non_blocking=True)
            engine.step_sharded_staged()
            for k in range(n_chunks):
                outs[k].copy_(engine.shards[k][3], non_blocking=True)
    else:
        fn = lambda: engine.step_sharded(grad_blocks, gather_blocks, host_grads=grads, host_params=outs)
    steps = max(1, min(args.steps, args.e2e_steps))
    for _ in range(2):
        fn()
    ms = timed(fn, steps) / steps
    ctl = engine.read_control()
    if ctl.status:
        raise SystemExit(f'bench e2e: status {ctl.status}')
    return {
        'value': total / (ms * 1e-3) / 1e9, 'unit': 'Gparams/s', 'ms_per_step': ms, 'steps': steps,
        'h2d_bytes_per_step': n_chunks * in_elems * 2 * world, 'd2h_bytes_per_step': n_chunks * shard * 2 * world,
        'conservative_ms_per_step': conservative_ms,
        'api': ('ChunkStepEngine.step_from_host' + ('' if conservative_ms is None else '(speculative=True)')) if world == 1 else
               ('ChunkStepEngine.step_sharded_p2p(host_grads=, host_params=)' if args.collective in ('p2p', 'p2p-fused', 'p2p-overlap') else
                'ChunkStepEngine.step_sharded_single_pass(host_grads=, host_params=)' if args.collective == 'mm' else
                'H2D into the gradient slab + ChunkStepEngine.step_sharded_staged + D2H of the shards'
                if args.collective == 'staged' else 'ChunkStepEngine.step_sharded(host_grads=, host_params=)'),
        'h2d_gbs_per_gpu': n_chunks * in_elems * 2 / (ms * 1e-3) / 1e9,
        'pinned_on_gpu_numa_node': bool(numa_cpus),
        'note': ('pinned fp16 gradients in, updated fp16 parameters out; fp32 master and moments stay in HBM; the host '
                 f'side is a pool of {pool} pinned buffers per direction reused over the chunks (every byte is still moved '
                 'every step)' + ('' if world == 1 else '; every rank uploads its own full-size gradient block of every '
                                  'chunk, so this leg is bound by PCIe and host memory, not by the step')),
    }


# ------------------------------------------------------------------------------------------------------
# residency modes of the wrapper (a secondary measurement: one training iteration, not the contract line)
# ------------------------------------------------------------------------------------------------------


def run_probe_rate(args):
    """``--workload probe-rate``: the inf/nan probe alone, load/store form (``probe_variant`` 0) against the bulk-copy
    ring (2), on one contiguous fp16 array of growing size (``elx_grad_check``) and on a table of 47 chunks of 32 Mi
    elements (``elx_grad_check_multi``).  Minimum of 7 launches after 3 warm-up launches, CUDA events around each
    launch.  One JSON line.  Synthetic data (zeros: the probe's work does not depend on the values)."""
    from elixir_b200 import kernels as K
    device = torch.device('cuda', 0)
    torch.cuda.set_device(device)

    def best_ms(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(7):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        return min(times)

    ctl = K.ControlBlock(device)
    n_chunks, chunk = 47, 32 * 1024 * 1024
    flat = torch.zeros(int(25.77e9) // 2, dtype=torch.float16, device=device)
    rows = []
    try:
        for gb in (0.016, 0.067, 0.268, 1.0, 3.15, 12.9, 25.77):
            g = flat[:int(gb * 1e9) // 2]
            row = {'form': 'one array', 'bytes': g.numel() * 2}
            for variant, name in ((0, 'loads'), (2, 'ring')):
                K.set_tuning(probe_variant=variant)
                ms = best_ms(lambda: K.grad_check(g, ctl=ctl))
                row[name] = {'ms': ms, 'TBs': g.numel() * 2 / ms / 1e9}
            rows.append(row)
        table = K.ChunkTable(device, torch.float16)
        stub = torch.zeros(chunk, dtype=torch.float32, device=device)    # the probe never touches the fp32 arrays
        for c in range(n_chunks):
            table.add_chunk(stub, stub, stub, flat[c * chunk:(c + 1) * chunk], n_valid=chunk - (5 if c % 3 == 0 else 0),
                            segments=[(0, chunk - 5, 0)])
        table.finalize()
        flags = torch.zeros(n_chunks, dtype=torch.int32, device=device)
        row = {'form': f'table of {n_chunks} chunks', 'bytes': n_chunks * chunk * 2}
        for variant, name in ((0, 'loads'), (2, 'ring')):
            K.set_tuning(probe_variant=variant)
            ms = best_ms(lambda: K.grad_check_multi(table, ctl, chunk_flags=flags))
            row[name] = {'ms': ms, 'TBs': n_chunks * chunk * 2 / ms / 1e9}
        rows.append(row)
    finally:
        K.set_tuning(probe_variant=-1)
    c = ctl.read()
    assert c.found_inf == 0 and c.status == 0 and int(flags.sum().item()) == 0
    peak, peak_kind = load_peaks()
    print(json.dumps({'workload': 'probe-rate', 'unit': 'TB/s', 'hbm_copy_peak_gbs': peak, 'peak_kind': peak_kind, 'rows': rows}))


def run_residency(args):
    """``--workload residency``: time one training iteration (forward, backward, optimizer step) of a stack of MLP
    blocks behind ``ElixirModule`` / ``ElixirOptimizer`` under the three ways of keeping chunks resident — ``all``: a
    replica-cache block per chunk; ``fifo``: ``--blocks`` blocks, chunks fetched sub-module by sub-module on the main
    stream; ``prefetch``: the same blocks, Belady's rule on the learnt access trace, gathers ahead and reduces on
    side streams.  One chunk holds one block of the stack.  Prints one JSON line per mode (rank 0): milliseconds per
    iteration (CUDA events, max over ranks), peak device memory, fetch counters.  Synthetic data, random weights."""
    import gc
    import torch.distributed as dist
    import torch.nn as nn
    from elixir_b200.optim import HybridAdam
    from elixir_b200.wrapper import ElixirModule, ElixirOptimizer, simple_plan

    class Block(nn.Module):

        def __init__(self, hidden):
            super().__init__()
            self.up = nn.Linear(hidden, 4 * hidden)
            self.down = nn.Linear(4 * hidden, hidden)

        def forward(self, x):
            return x + self.down(torch.nn.functional.gelu(self.up(x)))

    class Stack(nn.Module):

        def __init__(self, layers, hidden):
            super().__init__()
            self.blocks = nn.ModuleList(Block(hidden) for _ in range(layers))

        def forward(self, x):
            for block in self.blocks:
                x = block(x)
            return x.float().pow(2).mean()

    rank, world = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1))
    device = torch.device('cuda', int(os.environ.get('LOCAL_RANK', 0)))
    torch.cuda.set_device(device)
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29577')
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=device)
    group = dist.group.WORLD
    for mode in ('all', 'fifo', 'prefetch'):
        torch.manual_seed(0)
        with torch.device(device):
            model = Stack(args.layers, args.hidden).to(torch.float16)
        per_block = sum(p.numel() for p in model.blocks[0].parameters())
        blocks = None if mode == 'all' else args.blocks
        sr = simple_plan(model, world, unified_dtype=torch.float16, shard_device=device, chunk_size=per_block,
                         public_block_number=blocks)
        emodel = ElixirModule(model, sr, group, prefetch=(mode != 'fifo'), dtype=torch.float16)
        eoptim = ElixirOptimizer(emodel, HybridAdam(model.parameters(), lr=1e-4), initial_scale=1024.0)
        x = torch.randn(args.tokens, args.hidden, device=device, dtype=torch.float16)
        torch.cuda.reset_peak_memory_stats(device)
        rcache_gb = sr.chunk_group.rcache.public_space / 1e9

        def iteration():
            eoptim.zero_grad()
            eoptim.backward(emodel(x))
            eoptim.step()

        for _ in range(args.warmup):
            iteration()
        torch.cuda.synchronize(device)
        dist.barrier(group)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(args.steps):
            iteration()
        stop.record()
        torch.cuda.synchronize(device)
        ms = torch.tensor([start.elapsed_time(stop) / args.steps], device=device)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=group)
        eoptim.engine.check_status()
        if rank == 0:
            print(json.dumps(dict(workload='residency', mode=mode, ms_per_iteration=round(float(ms), 3), world=world,
                                  layers=args.layers, hidden=args.hidden, tokens=args.tokens, chunk_elems=per_block,
                                  chunks=len(emodel.param_chunks),
                                  blocks=len(emodel.param_chunks) if blocks is None else blocks,
                                  replica_cache_gb=round(rcache_gb, 2),
                                  peak_mem_gb=round(torch.cuda.max_memory_allocated(device) / 1e9, 2),
                                  fetch=dict(emodel.fetcher.stats) if emodel.scheduled else None)), flush=True)
        del emodel, eoptim, model, sr, iteration, x
        gc.collect()    # module <-> hook cycles keep the chunks alive otherwise
        torch.cuda.empty_cache()
    dist.barrier()
    dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------------
# CPU arms
# ------------------------------------------------------------------------------------------------------


def _cpu_inputs(chunks, chunk, scale, sigma, seed):
    sets = []
    for c in range(chunks):
        gen = torch.Generator().manual_seed(seed + c)
        master = torch.randn(chunk, generator=gen) * 0.02
        grad = (torch.randn(chunk, generator=gen) * sigma * scale).half()
        sets.append((master, grad))
    return sets


def cpu_torch_adamw(sets, scale, wd, steps):
    """The reference's CPU path with torch.optim.AdamW standing in for ColossalAI CPUAdam: finite check of
    the fp16 gradients, unscale to fp32, AdamW on the fp32 masters, fp16 copy-back."""
    params = [torch.nn.Parameter(m.clone()) for m, _ in sets]
    best = None
    for kwargs in (dict(foreach=True), dict(fused=True)):
        try:
            opt = torch.optim.AdamW(params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=wd, **kwargs)
        except (RuntimeError, TypeError):
            continue
        lowp = [g.clone() for _, g in sets]
        times = []
        for s in range(steps + 1):
            for buf, (_, g) in zip(lowp, sets):
                buf.copy_(g)
            t0 = time.perf_counter()
            overflow = any(not torch.isfinite(buf).all().item() for buf in lowp)
            if not overflow:
                for p, buf in zip(params, lowp):
                    p.grad = buf.float().div_(scale)
                opt.step()
            for p, buf in zip(params, lowp):
                buf.copy_(p.data)
            times.append(time.perf_counter() - t0)
        t = statistics.mean(times[1:])
        if best is None or t < best[0]:
            best = (t, 'torch.optim.AdamW(%s)' % ','.join(kwargs))
    return best


def cpu_oracle(sets, scale, wd, steps):
    from oracle import oracle as orc
    from elixir_b200 import kernels as K
    cs = orc.ChunkSet(torch.float16)
    lowp = []
    for master, g in sets:
        n = master.numel()
        buf = g.clone()
        cs.add_chunk(master.clone(), torch.zeros(n), torch.zeros(n), buf, n, [(0, n, 0)])
        lowp.append(buf)
    ctl = orc.new_ctl(scale)
    cfg = K.scaler_cfg(True)
    hyper = [K.hyper(weight_decay=wd)]
    times = []
    for s in range(steps + 1):
        for buf, (_, g) in zip(lowp, sets):
            buf.copy_(g)
        t0 = time.perf_counter()
        cs.step(ctl, cfg, hyper, probe=True, f64=False)
        times.append(time.perf_counter() - t0)
    return statistics.mean(times[1:]), orc.num_threads()


def cpu_baseline(args, chunk, scale, sigma, wd, steps, chunks):
    torch.set_num_threads(os.cpu_count())
    sets = _cpu_inputs(chunks, chunk, scale, sigma, args.seed)
    n = chunks * chunk
    t_torch, how = cpu_torch_adamw(sets, scale, wd, steps)
    t_orc, threads = cpu_oracle(sets, scale, wd, steps)
    best = min(t_torch, t_orc)
    return {
        'value': n / best / 1e9, 'unit': 'Gparams/s', 'cores': os.cpu_count(), 'kind': 'port',
        'sample': f'{chunks} chunks x {chunk} elements of the same workload, {steps} timed steps after 1 warm-up',
        'torch_adamw_gparams_per_s': n / t_torch / 1e9, 'torch_variant': how,
        'c_oracle_gparams_per_s': n / t_orc / 1e9, 'c_oracle_threads': threads,
        'note': 'ColossalAI CPUAdam/HybridAdam is not installable offline; torch.optim.AdamW on the host cores '
                'and the OpenMP C restatement of the same step stand in, the faster one is reported',
    }


def run_reference(args):
    """The reference's CPU implementation of the path on the host cores (rank 0 only)."""
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    world = args.gpus
    if world == 1:
        workload, total, chunk, scale, wd = 'gpt2xl_chunks_1gpu', GPT2XL_PARAMS, CHUNK_1GPU, 65536.0, 0.01
    else:
        workload, total, chunk, scale, wd = f'opt13b_chunks_sharded_w{world}', OPT13B_PARAMS, CHUNK_SHARDED, 1024.0, 0.0
    chunks = 4 if world == 1 else 1
    sample_chunk = chunk if world == 1 else chunk // 2
    torch.set_num_threads(os.cpu_count())
    sets = _cpu_inputs(chunks, sample_chunk, scale, 1e-3, args.seed)
    n = chunks * sample_chunk
    steps = max(1, min(args.steps, 5))
    t0 = time.perf_counter()
    t_torch, how = cpu_torch_adamw(sets, scale, wd, steps)
    t_orc, threads = cpu_oracle(sets, scale, wd, steps)
    best = min(t_torch, t_orc)
    value = n / best / 1e9
    line = {
        'impl': 'reference', 'metric': 'chunk Adam Gparams/s', 'value': value, 'unit': 'Gparams/s', 'n_gpus': world,
        'steps': steps, 'warmup': 1, 'ms_per_step': best * 1e3 * (total / n), 'higher_is_better': True,
        'scaling': 'weak' if world == 1 else 'strong', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': workload, 'params': total, 'chunk_elems': chunk,
                   'sampled_elements': n, 'note': 'ms_per_step is the sample time scaled to the full parameter count'},
        'cpu_baseline': {
            'value': value, 'unit': 'Gparams/s', 'cores': os.cpu_count(), 'kind': 'port',
            'sample': f'{chunks} chunks x {sample_chunk} elements, {steps} timed steps after 1 warm-up '
                      f'(wall {time.perf_counter() - t0:.1f} s)',
            'torch_adamw_gparams_per_s': n / t_torch / 1e9, 'torch_variant': how,
            'c_oracle_gparams_per_s': n / t_orc / 1e9, 'c_oracle_threads': threads,
        },
        'e2e': {'value': value, 'unit': 'Gparams/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=50)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--seed', type=int, default=0)
    ap.add_argument('--collective', default='auto', choices=['auto', 'p2p', 'p2p-fused', 'p2p-overlap', 'mm', 'staged', 'nccl'],
                    help='N > 1: p2p = pull reduce-scatter and push all-gather kernels over peer-mapped NVLink memory; '
                    'mm = ONE kernel per step that reduces, updates and gathers tile by tile through the NVLink switch '
                    '(multimem); p2p-fused = both collectives inside the in-place update kernel over peer-mapped memory, the '
                    'decision taken on the inputs first (two ranks); p2p-overlap = the p2p kernels with the decision taken on the inputs first, so that the update '
                    'of a chunk runs while the next one is reduced; staged = copy engines; nccl = NCCL on side streams; '
                    'auto = mm from 4 ranks on (where its two state sets fit), p2p-fused at 2 ranks, else p2p')
    ap.add_argument('--workload', default='auto', choices=['auto', 'opt66b_bf16', 'residency', 'probe-rate'],
                    help='N > 1: auto = OPT-13B-shaped fp16 chunk set; opt66b_bf16 = OPT-66B-shaped bf16 chunk set (8 GPUs); '
                    'residency = one training iteration of an MLP stack through the wrapper under three residency modes; '
                    'probe-rate = the inf/nan probe alone, load/store form against the bulk-copy ring (1 GPU)')
    ap.add_argument('--layers', type=int, default=12, help='residency workload: blocks of the stack (one chunk each)')
    ap.add_argument('--hidden', type=int, default=4096, help='residency workload: hidden size')
    ap.add_argument('--tokens', type=int, default=8192, help='residency workload: rows of the input')
    ap.add_argument('--blocks', type=int, default=3, help='residency workload: replica-cache blocks of the two scheduled modes')
    ap.add_argument('--chunk-elems', type=int, default=0, help='override the chunk size in elements (profiling cases)')
    ap.add_argument('--params', type=int, default=0, help='override the parameter count (smoke runs of a workload)')
    ap.add_argument('--pool', type=int, default=0,
                    help='N > 1: number of replicated blocks per slab (0 = one per chunk); chunk k uses block k %% pool')
    ap.add_argument('--step', choices=['single-pass', 'probe-update'], default='single-pass',
                    help='N = 1: single-pass = ONE update launch that also detects inf/nan, out of place between two sets '
                    'of master/moment arrays; probe-update = a probe launch over all gradient blocks, then the update in place')
    ap.add_argument('--landing', choices=['none', 'copy'], default='none',
                    help='N = 1: none = probe and update read the gradient blocks in place; copy = every block is first '
                    'copied into its shard by the reduce epilogue (probe fused), one launch per chunk')
    ap.add_argument('--ncu-traffic-bytes', type=float, default=0.0,
                    help='dram__bytes_read.sum + dram__bytes_write.sum of one update launch of this command, from an ncu '
                    'capture, to be reported as roofline.traffic')
    ap.add_argument('--land-streams', type=int, default=2,
                    help='N = 1: side streams the per-chunk landing launches alternate on')
    ap.add_argument('--pull-ctas', type=int, default=36,
                    help='p2p-overlap: CTAs of the pull kernel; the update kernel gets the remaining SMs')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-parity-check', action='store_true',
                    help='N > 1: skip the small sharded case that is checked against the CPU oracle before the warm-up')
    ap.add_argument('--no-e2e', action='store_true')
    ap.add_argument('--no-numa', action='store_true',
                    help='end-to-end leg: do not move to the CPUs of the GPU\'s NUMA node while the pinned buffers are allocated')
    ap.add_argument('--no-speculation', action='store_true',
                    help='N=1 end-to-end leg: only the step that updates nothing before the last gradient is probed')
    ap.add_argument('--shards', choices=['device', 'host', 'host-streamed'], default='device',
                    help="'host': optimizer state in pinned host memory, updated in place over PCIe by the kernel; "
                    "'host-streamed': the same state moved by the copy engines through device staging sets (N=1 only)")
    ap.add_argument('--e2e-steps', type=int, default=10)
    ap.add_argument('--tune', action='append', default=[], metavar='KNOB=VALUE',
                    help='launch-shape knob of the library (elx_set_tuning), for experiments; results do not depend on them')
    args = ap.parse_args()
    args.collective_was_auto = args.collective == 'auto'
    if args.collective_was_auto:
        plain = args.workload == 'auto' and not args.pool    # a block per chunk, fp16, no pooled slabs
        args.collective = 'mm' if plain and args.gpus >= 4 else 'p2p-fused' if plain and args.gpus == 2 else 'p2p'
    if args.workload == 'residency':
        run_residency(args)
    elif args.workload == 'probe-rate':
        run_probe_rate(args)
    elif args.impl == 'reference':
        run_reference(args)
    else:
        if args.warmup < 3:
            print('bench: warm-up raised to 3', file=sys.stderr)
            args.warmup = 3
        if args.tune:
            from elixir_b200 import kernels
            kernels.set_tuning(**{k: int(v) for k, v in (item.split('=', 1) for item in args.tune)})
        run_ours(args)


if __name__ == '__main__':
    main()
