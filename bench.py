#!/usr/bin/env python
"""Benchmark of the hash-map hot path: batched get + set (+ remove of the rows the set inserted) on the
hash-sharded CudaClosedHashmap of BASELINE.json configs[4].

Workload (default, strong scaling): 2^31 int64 keys drawn uniformly from [0, 2^62) mapped to float32[2] values at load
0.6, spread over the N GPUs by hash; a step is a get of 2^28 queries (80 % stored keys, 20 % absent), a set of 2^28
rows (80 % stored keys -> overwrite, 20 % new keys) and the removal of the rows that set inserted, which keeps the
load stationary; every rank submits 1/N of each batch.  N = 1 is the whole table on one GPU (114.5 GB of slots, worked
through in two passes per batch because it exceeds the 64 GiB the TLB covers); with N > 1 each rank routes its rows
to the owning shards over NVLink (sliced exchange) and gets the results back.  `--scaling weak` keeps 2^28 keys and
2^25-row batches PER GPU instead (N = 8 is then the same 2^31-key table).

  python bench.py [--gpus N] [--steps K] [--warmup W]            candidate (CUDA), one process per GPU
  python bench.py --impl reference ...                            the reference's own kernels on the host cores

One JSON line on stdout (rank 0).  Inputs are seeded and synthetic; nothing is read from disk except
MEASURED_PEAKS.json (the roofline denominator).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M62 = (1 << 62) - 1
KEY_BYTES, VALUE_BYTES = 8, 8
HIT_FRACTION = 0.8
LOAD_FACTOR = 0.6
N_BATCHES = 4          # distinct query/update batches rotated over the steps (each is larger than L2); 2 for huge batches
# DRAM bytes per operation of the kernels, dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture divided by
# the rows of the launch (profiles/k_*_c5_shard_2e26keys.md; the capture ran at 2^26 keys and 2^24 rows, traffic per row
# does not depend on the size once the table is much larger than L2)
TRAFFIC_BYTES_PER_OP = {"get": 169.6, "set": 206.9, "remove": 237.4}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["candidate", "reference"], default="candidate")
    ap.add_argument("--scaling", choices=["strong", "weak"], default="strong",
                    help="strong (default): --keys-log2 / --batch-log2 are TOTALS split over the GPUs; weak: per GPU")
    ap.add_argument("--keys-log2", type=int, default=None, help="stored keys: total 2^31 (strong) or 2^28 per GPU (weak)")
    ap.add_argument("--batch-log2", type=int, default=None, help="rows per operation and step: total 2^28 (strong) or 2^25 per GPU (weak)")
    ap.add_argument("--no-ref-gpu", action="store_true",
                    help="reference arm: skip the extra leg that runs the reference's kernels on the GPU")
    ap.add_argument("--no-peer", action="store_true",
                    help="multi-GPU: exchange rows with NCCL all-to-all instead of stores into the peers' memory")
    ap.add_argument("--no-pipeline", action="store_true",
                    help="multi-GPU: call get / set / remove one after the other instead of one pipelined submission")
    ap.add_argument("--send-blocks-per-sm", type=float, default=None,
                    help="multi-GPU: blocks per SM of the partition kernels while table kernels of another operation are "
                         "in flight (library default 3; 0 = one block per tile of 2048 rows, the whole grid at once)")
    ap.add_argument("--send-priority", type=int, default=None, choices=[-1, 0],
                    help="multi-GPU: priority of the stream the send stages run on (library default -1, high)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer (end-to-end) measurement")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-shard-point", action="store_true",
                    help="1 GPU, strong scaling: skip the extra leg on a 2^28-key table (the size the reference's kernels can hold)")
    ap.add_argument("--no-extras", action="store_true", help="1 GPU: skip the legs on BASELINE configs 1', 2, 3 and 4")
    ap.add_argument("--window-gib", type=float, default=0.0,
                    help="serve tables beyond the TLB's reach in windows of at most this many GiB (default: the library's 58)")
    ap.add_argument("--small-dok", action="store_true",
                    help="instead of the benchmark: one small pass over the DOK tensor and partition kernels (fused "
                         "get over selectors, to_sparse_coo, from_dense, partition scatter) on tables a few times L2; "
                         "the case to capture them under a profiler")
    ap.add_argument("--hw-probe", action="store_true",
                    help="instead of the benchmark: rate of random requests of 8..128 bytes over buffers of --probe-mib "
                         "MiB (what bounds every probing kernel); one JSON line")
    ap.add_argument("--probe-mib", type=int, nargs="+", default=[256, 1024, 4096, 16384, 65536, 73728, 81920, 98304, 116736])
    ap.add_argument("--probe-requests-log2", type=int, default=25)
    ap.add_argument("--probe-reps", type=int, default=5)
    ap.add_argument("--l2-fetch-granularity", type=int, default=0,
                    help="--hw-probe: cudaDeviceSetLimit(cudaLimitMaxL2FetchGranularity, N) for this process first (32/64/128)")
    args = ap.parse_args()
    if args.keys_log2 is None:
        args.keys_log2 = 31 if args.scaling == "strong" else 28
    if args.batch_log2 is None:
        args.batch_log2 = 28 if args.scaling == "strong" else 25
    return args


def sizes_per_gpu(args, world):
    """(stored keys, rows per operation and step) of ONE rank"""
    if args.scaling == "strong":
        return (1 << args.keys_log2) // world, (1 << args.batch_log2) // world
    return 1 << args.keys_log2, 1 << args.batch_log2


# ---------------------------------------------------------------------------------------------------------------
# byte model and peaks
# ---------------------------------------------------------------------------------------------------------------

def algorithmic_bytes(op, kb=KEY_BYTES, vb=VALUE_BYTES, hit=HIT_FRACTION):
    """Bytes one operation must move with the ideal layout (tag and value in one 32-byte sector)."""
    sectors = -(-(8 + vb) // 32)
    if op == "get":       # key in, value + flag out, one sector read per probe chain (hit: the bucket row, miss: one tag)
        return kb + vb + 1 + 32 * (hit * sectors + (1 - hit))
    if op == "set":       # key + value in, the bucket sector(s) and the key-row sector read and written back
        return kb + vb + 2 * 32 * -(-(8 + vb + kb) // 32)
    if op == "remove":    # key in, flag out, the tag sector read and written back
        return kb + 1 + 2 * 32
    raise ValueError(op)


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


# ---------------------------------------------------------------------------------------------------------------
# synthetic keys: a bijection of [0, 2^62) makes every key index a distinct, uniformly spread key
# ---------------------------------------------------------------------------------------------------------------

def mix62_torch(x):
    x = (x * 0x2545F4914F6CDD1D) & M62
    x = x ^ (x >> 29)
    x = (x * 0x1B03738712FAD5C9) & M62
    x = x ^ (x >> 32)
    return x


def mix62_numpy(x):
    x = x.astype(np.uint64)
    m = np.uint64(M62)
    x = (x * np.uint64(0x2545F4914F6CDD1D)) & m
    x = x ^ (x >> np.uint64(29))
    x = (x * np.uint64(0x1B03738712FAD5C9)) & m
    x = x ^ (x >> np.uint64(32))
    return x.astype(np.int64)


def value_of_index(idx, xp):
    """float32[2] value stored for key index idx (lets the bench verify what a get returns)"""
    a = (idx & 0xFFFF)
    b = ((idx >> 16) & 0xFF)
    if xp is np:
        return np.stack([a, b], axis=1).astype(np.float32)
    return xp.stack([a, b], dim=1).float()


def fixed_parameters():
    """Explicit hash parameters, identical on every rank: one draw of the reference's generator (numpy seed 2024)
    for a table of 2^28 / 0.6 buckets."""
    return dict(prime1=[825411893], prime2=[131956765728754273], alpha1=[808106522], alpha2=[408516131],
                beta1=[188156349], beta2=[614383798])


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.thread = [], None, None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "25"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
                for name, cell in zip(names, r[4:8]):
                    if cell.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                pass
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------------------
# CPU arm: the reference's own kernels compiled for the host (oracle/_ref), else the C restatement
# ---------------------------------------------------------------------------------------------------------------

def cpu_arm(steps, warmup, sample_keys_log2=24, sample_batch_log2=22, budget_s=None):
    """One step = get(q) + set(q) + remove(inserted) on a table of 2^sample_keys_log2 keys at load 0.6, all host
    threads.  Returns (Mops/s over get+set rows, description dict)."""
    from oracle import port, ref
    cores = len(os.sched_getaffinity(0))
    n_keys, q = 1 << sample_keys_log2, 1 << sample_batch_log2
    nb = int(n_keys / LOAD_FACTOR)
    params = {k: np.asarray(v, dtype=np.int64) for k, v in fixed_parameters().items()}
    params["key_perm"] = np.zeros(1, dtype=np.int64)
    use_ref = os.path.exists(ref.map_lib_path("i64x1_f32x2"))
    if use_ref:
        table = ref.RefMap(nb, np.int64, 1, np.float32, 2, params, n_threads=cores)
        do_set, do_get, do_remove = table.set, table.get, table.remove
        kind = "reference"
    else:
        table = port.OracleHashmap(n_buckets=nb, n_threads=cores, **{k: v for k, v in params.items() if k != "key_perm"})
        table._keys, table._values = np.zeros((nb, 1), np.int64), np.zeros((nb, 2), np.float32)
        do_set, do_get, do_remove = table.set_rows, table._kernel_get, table.remove_rows
        kind = "port"
    idx = np.arange(n_keys, dtype=np.int64)
    for lo in range(0, n_keys, 1 << 22):
        part = idx[lo:lo + (1 << 22)]
        do_set(mix62_numpy(part)[:, None], value_of_index(part, np))
    n_hit = int(q * HIT_FRACTION)
    batches = []
    for b in range(2):
        rng = np.random.default_rng(b)
        hit_idx = (np.arange(n_hit, dtype=np.int64) * 7919 + 104729 * (b + 1)) % n_keys
        miss_idx = (1 << 40) + (b << 32) + np.arange(q - n_hit, dtype=np.int64)
        new_idx = (1 << 41) + (b << 32) + np.arange(q - n_hit, dtype=np.int64)
        perm = rng.permutation(q)
        gq = mix62_numpy(np.concatenate([hit_idx, miss_idx]))[perm][:, None]
        sk_idx = np.concatenate([hit_idx, new_idx])[perm]
        batches.append((gq, mix62_numpy(sk_idx)[:, None], value_of_index(sk_idx, np), mix62_numpy(new_idx)[:, None]))

    def step(b):
        gq, sk, sv, fresh = batches[b % 2]
        do_get(gq)
        do_set(sk, sv)
        do_remove(fresh)

    for s in range(warmup):
        step(s)
    t0 = time.perf_counter()
    done = 0
    for s in range(steps):
        step(s)
        done += 1
        if budget_s is not None and time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    mops = done * 2 * q / dt / 1e6
    desc = {"value": mops, "unit": "Mops/s", "cores": cores, "kind": kind,
            "sample": f"table of 2^{sample_keys_log2} keys at load {LOAD_FACTOR}, {done} steps of get 2^{sample_batch_log2} + "
                      f"set 2^{sample_batch_log2} + remove of the inserted 20 %, kernels only (no Python-side pre-get / unique)"}
    return mops, dt / max(done, 1) * 1e3, desc


SHARD_POINT_KEYS_LOG2, SHARD_POINT_BATCH_LOG2 = 28, 25      # the largest power-of-two table the reference's kernels hold


def make_batches(torch, device, n_batches, q, total_keys, rank, keep_idx=(0,)):
    """Seeded batches of one rank: get keys (80 % stored anywhere in the table, 20 % absent), set rows (80 % stored ->
    overwrite, 20 % new) and the new keys (removed again at the end of a step)."""
    n_hit = int(q * HIT_FRACTION)
    g = torch.Generator(device=device).manual_seed(1234 + rank)
    batches = []
    for b in range(n_batches):
        j = torch.arange(n_hit, device=device, dtype=torch.long)
        hit_idx = (j * 7919 + 104729 * (b + 1) + 15485863 * rank) % total_keys
        del j
        base = (b << 34) + (rank << 30)
        tail = torch.arange(q - n_hit, device=device, dtype=torch.long)
        miss_idx, new_idx = (1 << 40) + base + tail, (1 << 41) + base + tail
        del tail
        perm = torch.randperm(q, device=device, generator=g)
        get_idx = torch.cat([hit_idx, miss_idx])[perm]
        del miss_idx
        set_idx = torch.cat([hit_idx, new_idx])[perm]
        del hit_idx, perm
        d = {"get_keys": mix62_torch(get_idx)[:, None].contiguous(),
             "set_keys": mix62_torch(set_idx)[:, None].contiguous(), "set_values": value_of_index(set_idx, torch).contiguous(),
             "fresh_keys": mix62_torch(new_idx)[:, None].contiguous()}
        if b in keep_idx:
            d["get_idx"], d["set_idx"] = get_idx, set_idx
        del get_idx, set_idx, new_idx
        batches.append(d)
    return batches


def reference_kernels_on_gpu(steps=5, warmup=3):
    """The reference's own get / set / remove kernels (its kernel text compiled ahead of time by nvcc, since CuPy is
    not available) on cuda:0, on a table of 2^28 keys at load 0.6 with 2^25-row batches -- one shard of the 8-GPU
    configuration, and the largest power-of-two size its 32-bit bucket indices hold (closed_hashmap_impl_class.cu:184)
    -- with the same batch construction and operation order as the candidate's `shard_point` leg.  Kernels only: the
    reference's Python bookkeeping around them (a pre-get, a row-sort unique and host synchronisations per set; a
    unique per remove) is left out, which favours the reference; `api_path` adds it back.
    Returns a dict for the JSON line, or a reason string when it cannot run here."""
    try:
        import torch
        from oracle import ref_gpu
    except Exception as exc:                                    # pragma: no cover
        return f"import failed: {exc}"
    if not torch.cuda.is_available():
        return "no GPU"
    if not ref_gpu.available(torch.int64, 1, torch.float32, 2):
        return "oracle/_ref/refgpu_map_i64x1_f32x2.so not built"
    device = torch.device("cuda", 0)
    n_keys, q = 1 << SHARD_POINT_KEYS_LOG2, 1 << SHARD_POINT_BATCH_LOG2
    nb = int(n_keys / LOAD_FACTOR)
    if nb * 2 > ref_gpu.RefGpuMap.MAX_ELEMENTS:
        return "table beyond the reference's 32-bit bucket indices"
    table = ref_gpu.RefGpuMap(nb, torch.int64, 1, torch.float32, 2, dict(fixed_parameters(), key_perm=[0]), device)
    chunk = min(n_keys, 1 << 25)
    for lo in range(0, n_keys, chunk):
        idx = torch.arange(lo, lo + chunk, device=device, dtype=torch.long)
        table.set(mix62_torch(idx)[:, None].contiguous(), value_of_index(idx, torch).contiguous())
    batches = make_batches(torch, device, N_BATCHES, q, n_keys, 0)

    def step(b, events=None):
        d = batches[b % N_BATCHES]
        marks = []
        for fn in (lambda: table.get(d["get_keys"]), lambda: table.set(d["set_keys"], d["set_values"]),
                   lambda: table.remove(d["fresh_keys"]), None):
            if events is not None:
                marks.append(torch.cuda.Event(enable_timing=True)); marks[-1].record()
            if fn is not None:
                fn()
        if events is not None:
            events.append(marks)

    values, found = table.get(batches[0]["get_keys"])
    expect = batches[0]["get_idx"] < (1 << 40)
    ok = bool(torch.equal(found, expect)) and bool(torch.equal(values[expect], value_of_index(batches[0]["get_idx"][expect], torch)))
    for s in range(warmup):
        step(s)
    torch.cuda.synchronize()
    events = []
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for s in range(steps):
        step(warmup + s, events)
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / steps
    phase = [sum(m[i].elapsed_time(m[i + 1]) for m in events) / steps for i in range(3)]

    # the same step the way a user of the reference calls it: with the Python bookkeeping of its set / remove
    # (pre-get, row-wise unique, host read of n_elements) around the kernels
    def api_step(b):
        d = batches[b % N_BATCHES]
        table.get(d["get_keys"])
        table.api_set(d["set_keys"], d["set_values"], rehash_threshold=0.95)
        table.api_remove(d["fresh_keys"])

    table.n_elements = torch.tensor(n_keys, device=device)
    api_step(0)
    torch.cuda.synchronize()
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    api_steps = 3
    a0.record()
    for s in range(api_steps):
        api_step(1 + s)
    a1.record()
    torch.cuda.synchronize()
    api_ms = a0.elapsed_time(a1) / api_steps
    live = int(((table.all_uuids != -1) & (table.all_uuids != -3)).sum().item())
    return {"value": 2 * q / (ms * 1e-3) / 1e6, "unit": "Mops/s", "ms_per_step": ms,
            "keys": n_keys, "batch": q,
            "get_ms": phase[0], "set_ms": phase[1], "remove_ms": phase[2], "steps": steps, "results_ok": ok,
            "live_keys_after": live, "live_keys_expected": n_keys,
            "api_path": {"value": 2 * q / (api_ms * 1e-3) / 1e6, "unit": "Mops/s", "ms_per_step": api_ms, "steps": api_steps,
                         "what": "the same kernels with the reference's Python bookkeeping restated around them "
                                 "(cuda_closed_hashmap.py:321-384, 423-454: pre-get + unique(dim=0) + n_elements.item() "
                                 "per set, unique(dim=0) per remove), i.e. what a caller of the reference API pays"},
            "what": "the reference's closed_hashmap_get/set/remove kernels (closed_hashmap_impl.cu), nvcc -O3 for sm_100a, "
                    "launched like closed_hashmap_impl.py does, incl. its output allocation and fallback fill; "
                    "no Python-side pre-get / unique / rehash logic; 2^28 keys, 2^25-row batches (compare with the "
                    "candidate's shard_point)"}


CPU_SAMPLE_KEYS_LOG2, CPU_SAMPLE_BATCH_LOG2 = 24, 22


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    mops, ms, desc = cpu_arm(args.steps, args.warmup, CPU_SAMPLE_KEYS_LOG2, CPU_SAMPLE_BATCH_LOG2)
    gpu_leg = None if args.no_ref_gpu else reference_kernels_on_gpu()
    config = workload_config(args, world=args.gpus)
    # what this arm really ran: a bounded sample of the workload on the host cores
    config.update({"sample_of_workload": True, "sample_keys": 1 << CPU_SAMPLE_KEYS_LOG2, "sample_batch": 1 << CPU_SAMPLE_BATCH_LOG2,
                   "sample": desc["sample"]})
    line = {
        "impl": "reference", "metric": "hashmap get/set Mops/s", "value": mops, "unit": "Mops/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": "int64", "data": "synthetic",
        "config": config,
        "cpu_baseline": desc,
        "e2e": {"value": mops, "unit": "Mops/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        # extra: the same reference kernel text run on this box's GPU (kernel-only, 1 GPU); not the line's value
        "reference_kernels_gpu": gpu_leg,
    }
    print(json.dumps(line))


def workload_config(args, world):
    n_keys, q = sizes_per_gpu(args, world)
    n_batches = N_BATCHES if q < (1 << 27) else 2
    tuning = {}
    if getattr(args, "send_blocks_per_sm", None) is not None:
        tuning["send_blocks_per_sm"] = args.send_blocks_per_sm
    if getattr(args, "send_priority", None) is not None:
        tuning["send_priority"] = args.send_priority
    return {
        **tuning,
        "workload": "BASELINE configs[4]: hash-sharded CudaClosedHashmap, int64 keys uniform in [0,2^62) -> float32[2], "
                    f"{n_keys * world} keys in total ({n_keys} per GPU) at load {LOAD_FACTOR}; a step = get of {q * world} rows "
                    f"(80% hits) + set of {q * world} rows (80% overwrite, 20% insert) + remove of the inserted rows, "
                    f"{q} rows per GPU and operation",
        "total_keys": n_keys * world, "total_batch": q * world,
        "keys_per_gpu": n_keys, "buckets_per_gpu": int(n_keys / LOAD_FACTOR),
        "batch_per_gpu": q, "shards": world,
        "l2_policy": f"inputs larger than L2: {n_batches} rotating batches of {q * 8 >> 20} MiB keys per GPU, "
                     f"table {(int(n_keys / LOAD_FACTOR) * 32) >> 20} MiB per GPU",
        "parallelism": ("single GPU" if world == 1 else
                        f"hash-sharded x{world}, " + ("NCCL all-to-all" if getattr(args, "no_peer", False) else
                                                      "rows stored into fixed slices of the owners' memory over NVLink "
                                                      "(sliced exchange, no host waits)")),
    }


# ---------------------------------------------------------------------------------------------------------------
# candidate arm
# ---------------------------------------------------------------------------------------------------------------

def build_table(torch, table, n_keys, rank, device):
    """rank r inserts key indices [r * n_keys, (r + 1) * n_keys), routed to their owners (untimed)"""
    chunk = min(n_keys, 1 << 25)
    for lo in range(rank * n_keys, (rank + 1) * n_keys, chunk):
        idx = torch.arange(lo, lo + chunk, device=device, dtype=torch.long)
        table.set(mix62_torch(idx)[:, None], value_of_index(idx, torch), assume_unique=True)


def time_steps(torch, step, steps, first):
    """K sequential steps with per-operation CUDA events -> (ms per step, [get, set, remove] ms)"""
    events = []
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for s in range(steps):
        step(first + s, events)
    t1.record()
    torch.cuda.synchronize()
    phase = [0.0, 0.0, 0.0]
    for s in range(steps):
        e = events[4 * s: 4 * s + 4]
        for i in range(3):
            phase[i] += e[i].elapsed_time(e[i + 1]) / steps
    return t0.elapsed_time(t1) / steps, phase


def random_request_rate(torch, L, buf, nbytes, device, n_reads=1 << 26):
    """G random 16-byte reads per second over buf[0, nbytes): the ceiling of any probing kernel on that range"""
    lib = L.lib()
    lib.dok_diag_random_reads(L.ptr(buf), nbytes, n_reads, 1, None, L.stream_ptr(device))
    r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    r0.record()
    for rep in range(3):
        lib.dok_diag_random_reads(L.ptr(buf), nbytes, n_reads, 100 + rep, None, L.stream_ptr(device))
    r1.record()
    torch.cuda.synchronize()
    return 3 * n_reads / (r0.elapsed_time(r1) * 1e-3) / 1e9


def shard_point(torch, device):
    """This library's kernels on the table size the reference's kernels can hold (2^28 keys, 2^25-row batches, one GPU,
    device-resident): the leg to put beside `reference_kernels_gpu` of the reference arm."""
    from doksparse_b200 import CudaClosedHashmap
    n_keys, q = 1 << SHARD_POINT_KEYS_LOG2, 1 << SHARD_POINT_BATCH_LOG2
    table = CudaClosedHashmap(n_buckets=int(n_keys / LOAD_FACTOR), device=device, rehash_threshold=0.95, **fixed_parameters())
    build_table(torch, table, n_keys, 0, device)
    batches = make_batches(torch, device, N_BATCHES, q, n_keys, 0)

    def step(b, events=None):
        d = batches[b % N_BATCHES]
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        marks[0].record()
        values, found = table.get(d["get_keys"])
        marks[1].record()
        table.set(d["set_keys"], d["set_values"])
        marks[2].record()
        table.remove_rows(d["fresh_keys"])
        marks[3].record()
        if events is not None:
            events.extend(marks)
        return values, found

    values, found = step(0)
    expect = batches[0]["get_idx"] < (1 << 40)
    ok = bool(torch.equal(found, expect)) and bool(torch.equal(values[expect], value_of_index(batches[0]["get_idx"][expect], torch)))
    for s in range(1, 4):
        step(s)
    torch.cuda.synchronize()
    ms, phase = time_steps(torch, step, 10, 4)

    # the same step as the drop-in API is called: remove() makes the keys unique first, as the reference's does
    # (cuda_closed_hashmap.py:423-454 of the reference); compare with reference_kernels_gpu.api_path
    def api_step(b):
        d = batches[b % N_BATCHES]
        table.get(d["get_keys"])
        table.set(d["set_keys"], d["set_values"])
        table.remove(d["fresh_keys"])

    for s in range(3):
        api_step(s)
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a0.record()
    for s in range(5):
        api_step(3 + s)
    a1.record()
    torch.cuda.synchronize()
    api_ms = a0.elapsed_time(a1) / 5
    # load 0.5, the point the north-star is worded on: the same keys in a table of 2 * n_keys buckets
    half = CudaClosedHashmap(n_buckets=2 * n_keys, device=device, rehash_threshold=0.95, **fixed_parameters())
    build_table(torch, half, n_keys, 0, device)
    for s in range(3):
        half.get(batches[s % N_BATCHES]["get_keys"])
    h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    h0.record()
    for s in range(8):
        half.get(batches[s % N_BATCHES]["get_keys"])
    h1.record()
    torch.cuda.synchronize()
    get_half_ms = h0.elapsed_time(h1) / 8
    probes, _ = table.probe_stats(batches[0]["get_keys"])
    probes_half, _ = half.probe_stats(batches[0]["get_keys"])
    peak, _ = measured_peak_gbs()
    return {"keys": n_keys, "batch": q, "value": 2 * q / (ms * 1e-3) / 1e6, "unit": "Mops/s", "ms_per_step": ms,
            "get_ms": phase[0], "set_ms": phase[1], "remove_ms": phase[2], "results_ok": ok,
            "api_path": {"value": 2 * q / (api_ms * 1e-3) / 1e6, "unit": "Mops/s", "ms_per_step": api_ms, "steps": 5,
                         "what": "get, set, remove() with its unique-keys pass, as the drop-in API is called"},
            "get_frac": algorithmic_bytes("get") * q / (phase[0] * 1e-3) / 1e9 / peak,
            "set_frac": algorithmic_bytes("set") * q / (phase[1] * 1e-3) / 1e9 / peak,
            "remove_frac": algorithmic_bytes("remove") * (q - int(q * HIT_FRACTION)) / (phase[2] * 1e-3) / 1e9 / peak,
            "mean_probe_groups_load_0.6": probes,
            "get_load_0.5": {"ms": get_half_ms, "mops": q / (get_half_ms * 1e-3) / 1e6, "mean_probe_groups": probes_half,
                             "frac": algorithmic_bytes("get") * q / (get_half_ms * 1e-3) / 1e9 / peak},
            "what": "one shard of the 8-GPU configuration on one GPU, device-resident, operations called one after the "
                    "other; compare with reference_kernels_gpu of the reference arm (same table, same batches)"}


def run_candidate(args):
    import torch
    import torch.distributed as dist
    from doksparse_b200 import _lib as L
    from doksparse_b200.sharded import ShardedClosedHashmap

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"        # keep NCCL's banner off stdout: one JSON line only
        # the small collectives of the exchange (fences) must not queue behind the big probing grids
        os.environ.setdefault("TORCH_NCCL_HIGH_PRIORITY", "1")
        dist.init_process_group("nccl", device_id=device)
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run"
    if args.send_blocks_per_sm is not None:
        from doksparse_b200.sharded import CudaShardOps
        CudaShardOps.OVERLAPPED_ROUTING_BLOCKS_PER_SM = args.send_blocks_per_sm
    if args.send_priority is not None:
        ShardedClosedHashmap.SEND_STREAM_PRIORITY = args.send_priority

    n_keys, q = sizes_per_gpu(args, world)
    total_keys = n_keys * world
    nb = int(n_keys / LOAD_FACTOR)
    n_batches = N_BATCHES if q < (1 << 27) else 2
    if args.window_gib > 0:
        L.check(L.lib().dok_set_window_bytes(72 << 30, int(args.window_gib * (1 << 30))), "dok_set_window_bytes")
    # rows of a batch go straight into fixed slices of the owners' memory over NVLink; --no-peer keeps the NCCL
    # all-to-all exchange
    peer_rows = 0 if (world == 1 or args.no_peer) else q
    table = ShardedClosedHashmap(nb, device=device, rehash_threshold=0.95, peer_capacity_rows=peer_rows, **fixed_parameters())
    build_table(torch, table, n_keys, rank, device)
    assert table.n_elements == total_keys, "build lost keys"
    batches = make_batches(torch, device, n_batches, q, total_keys, rank)
    n_hit = int(q * HIT_FRACTION)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    pipelined = world > 1 and not args.no_peer and not args.no_pipeline

    def step(b, events=None):
        d = batches[b % n_batches]
        if pipelined and events is None:
            # one submission per step, not waited for: the host only enqueues, the send stage of each operation
            # overlaps the table work of the one before, also across steps (the timed loop waits once, at its end)
            (values, found), _, _ = table.run([("get", d["get_keys"]), ("set", d["set_keys"], d["set_values"]),
                                               ("remove", d["fresh_keys"])], wait=False)
            return values, found
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        marks[0].record()
        values, found = table.get(d["get_keys"])
        marks[1].record()
        table.set(d["set_keys"], d["set_values"])
        marks[2].record()
        table.remove(d["fresh_keys"])
        marks[3].record()
        if events is not None:
            events.extend(marks)
        return values, found

    # ---- correctness of what is being timed (first batch, before any timing): every operation against what the
    # synthetic data says it must return, through the same calls (and, with several GPUs, the same exchange)
    d0 = batches[0]
    values, found = step(0)
    if pipelined:
        table.wait()
    expect_found = d0["get_idx"] < (1 << 40)
    checks = {"found_flags_ok": bool(torch.equal(found, expect_found)),
              "hit_values_ok": bool(torch.equal(values[expect_found], value_of_index(d0["get_idx"][expect_found], torch))),
              "miss_values_zero": bool((values[~expect_found] == 0).all()),
              "n_elements_stationary": table.n_elements == total_keys}
    del values, found
    marked = d0["set_values"] + 0.5                                   # values no other row carries
    table.set(d0["set_keys"], marked)
    back, back_found = table.get(d0["set_keys"])
    checks["set_then_get_returns_set_values"] = bool(back_found.all()) and bool(torch.equal(back, marked))
    checks["n_elements_after_insert"] = table.n_elements == total_keys + (q - n_hit) * world
    checks["remove_reports_every_inserted_row"] = bool(table.remove(d0["fresh_keys"]).all())
    checks["second_remove_reports_none"] = not bool(table.remove(d0["fresh_keys"]).any())
    stored = d0["set_idx"] < (1 << 40)
    table.set(d0["set_keys"][stored], d0["set_values"][stored])       # the original values back
    if world > 1 and not args.no_peer:
        # a batch that does not fit its slices: skipped by every rank on the device, repeated over the all-to-all exchange
        (v_over, f_over), = table.run([("get", d0["get_keys"])], _force_overflow=True)
        checks["overflow_fallback_ok"] = bool(torch.equal(f_over, expect_found)) and bool(
            torch.equal(v_over[expect_found], value_of_index(d0["get_idx"][expect_found], torch)))
        del v_over, f_over
    checks["n_elements_restored"] = table.n_elements == total_keys
    del back, back_found, marked, stored, expect_found

    sampler = ClockSampler(local_rank) if rank == 0 else None      # started early: its start-up must not fall into the timed region
    for s in range(1, args.warmup):
        step(s)
    if pipelined:
        table.wait()
    if sampler:
        time.sleep(0.5)
        sampler.rows.clear()

    exchange_phases = None
    # ---- timed region: exactly K steps, device-resident inputs
    launches0 = L.lib().dok_launch_count()
    events = []
    barrier()
    t_start, t_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    host_t0 = time.perf_counter()
    for s in range(args.steps):
        step(s + args.warmup, None if pipelined else events)
    host_enqueue_ms = (time.perf_counter() - host_t0) * 1e3 / args.steps      # host time per step before the final wait
    if pipelined:
        table.wait()
    t_stop.record()
    barrier()
    launches = L.lib().dok_launch_count() - launches0
    clocks = sampler.stop() if sampler else None
    elapsed_ms = torch.tensor([t_start.elapsed_time(t_stop)], device=device)
    phase_steps = args.steps
    if pipelined:
        # the timed steps were pipelined submissions; the per-operation times come from a short separate pass that
        # calls the operations one after the other (they add up to more than a pipelined step)
        phase_steps = 3
        step(0, [])                                   # warm the sequential path (allocator pools of the main stream)
        barrier()
        table.profile = []                            # stage boundaries of every operation, as CUDA events
        for s in range(phase_steps):
            step(s + 1, events)
        barrier()
        exchange_phases = table.phase_times()
        table.profile = None
    phase = torch.zeros(3, device=device)
    for s in range(phase_steps):
        e = events[4 * s: 4 * s + 4]
        phase += torch.tensor([e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2]), e[2].elapsed_time(e[3])], device=device)
    phase /= phase_steps
    if world > 1:
        dist.all_reduce(elapsed_ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(phase, op=dist.ReduceOp.MAX)
    elapsed_ms = float(elapsed_ms.item())
    get_ms, set_ms, remove_ms = (float(x) for x in phase.tolist())
    ms_per_step = elapsed_ms / args.steps
    ops_per_step = 2 * q * world                         # get rows + set rows over all GPUs
    value = ops_per_step / (ms_per_step * 1e-3) / 1e6

    # ---- end to end: host (pinned) buffers in, host buffers out, through the public API
    e2e = None
    if not args.no_e2e:
        names = ("get_keys", "set_keys", "set_values", "fresh_keys")
        host = []
        for d in batches[:2]:
            h = {}
            for k in names:
                h[k] = torch.empty(d[k].shape, dtype=d[k].dtype, pin_memory=True)
                h[k].copy_(d[k])
            host.append(h)
        out_values = torch.empty(q, 2, dtype=torch.float32, pin_memory=True)
        out_found = torch.empty(q, dtype=torch.bool, pin_memory=True)
        h2d = sum(host[0][k].numel() * host[0][k].element_size() for k in names)
        d2h = out_values.numel() * 4 + out_found.numel()

        # what the host link gives when every rank copies at once and nothing else runs: the bound of the e2e leg
        probe_src, probe_dst = host[0]["get_keys"], torch.empty_like(batches[0]["get_keys"])
        probe_dst.copy_(probe_src, non_blocking=True)
        barrier()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        for _ in range(4):
            probe_dst.copy_(probe_src, non_blocking=True)
        p1.record()
        torch.cuda.synchronize()
        probe_gbs = torch.tensor([4 * probe_src.numel() * 8 / (p0.elapsed_time(p1) * 1e-3) / 1e9], device=device)
        if world > 1:
            dist.all_reduce(probe_gbs, op=dist.ReduceOp.MIN)
        del probe_dst

        from doksparse_b200.host_batch import HostBatch
        # chunks of 4 Mi rows on three streams (copy in | kernels | copy out); routed batches use larger chunks
        pipe = HostBatch(table, device, chunk_rows=(1 << 22) if world == 1 else min(q, 1 << 23))

        def e2e_step(b):
            h = host[b % 2]
            pipe.run([("get", h["get_keys"], out_values, out_found), ("set", h["set_keys"], h["set_values"]),
                      ("remove_rows", h["fresh_keys"])])

        e2e_steps = max(3, min(args.steps, 10 if q < (1 << 27) else 4))
        e2e_step(0)
        pipe.join()
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        pipe.begin()
        for s in range(e2e_steps):
            e2e_step(s + 1)
        pipe.join()
        t1.record()
        barrier()
        last = e2e_steps % 2
        e2e_found = out_found.to(device)
        e2e_checks = {"e2e_found_ok": bool(torch.equal(e2e_found, batches[0]["get_idx"] < (1 << 40))) if last == 0 else
                      int(e2e_found.sum()) == n_hit}
        del e2e_found
        e_ms = torch.tensor([t0.elapsed_time(t1)], device=device)
        if world > 1:
            dist.all_reduce(e_ms, op=dist.ReduceOp.MAX)
        e2e = {"value": ops_per_step / (float(e_ms.item()) / e2e_steps * 1e-3) / 1e6, "unit": "Mops/s",
               "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world, "steps": e2e_steps,
               "how": "HostBatch: pinned host buffers in and out, chunked over copy-in / kernel / copy-out streams",
               "ms_per_step": float(e_ms.item()) / e2e_steps,
               "h2d_gbs_per_gpu": h2d / (float(e_ms.item()) / e2e_steps * 1e-3) / 1e9,
               "h2d_copy_only_gbs_per_gpu": float(probe_gbs.item()),   # all ranks copying at once, slowest rank
               **e2e_checks}
        del host, out_values, out_found, pipe

    # ---- what the hardware gives a probing kernel: independent random 16-byte reads over this GPU's slot array, over
    # all of it and over one window of it (tables beyond the TLB's reach are served window by window)
    local = table.ops.local
    slots = local._slots
    passes = L.lib().dok_table_passes(local._c_table())
    ceiling_whole = random_request_rate(torch, L, slots, slots.numel(), device)
    ceiling_window = ceiling_whole if passes <= 1 else random_request_rate(torch, L, slots, slots.numel() // passes, device)
    probe_len, _ = local.probe_stats(batches[0]["get_keys"][: 1 << 22]) if world == 1 else (None, None)

    # ---- roofline of the dominant kernel and of the other two
    peak, peak_source = measured_peak_gbs()
    local_rows = {"get": q, "set": q, "remove": q - n_hit}       # rows each GPU processes per step
    kernel_ms = {"get": get_ms, "set": set_ms, "remove": remove_ms}
    per_kernel = {}
    for op in ("get", "set", "remove"):
        achieved = algorithmic_bytes(op) * local_rows[op] / (kernel_ms[op] * 1e-3) / 1e9
        gops = local_rows[op] / (kernel_ms[op] * 1e-3) / 1e9
        per_kernel[op] = {"ms": kernel_ms[op], "mops_per_gpu": gops * 1e3, "bytes_per_op": algorithmic_bytes(op),
                          "achieved_gbs": achieved, "frac": achieved / peak,
                          "frac_of_random_request_ceiling": gops / ceiling_window}
        if TRAFFIC_BYTES_PER_OP.get(op) and world == 1:
            # what DRAM really moves (ncu: a whole 128-byte line per probed group), as a rate and against the peak;
            # a table served in several passes reads the batch once per pass
            extra = (passes - 1) * (KEY_BYTES if op != "set" else KEY_BYTES + VALUE_BYTES) if passes > 1 else 0
            dram = (TRAFFIC_BYTES_PER_OP[op] + extra) * local_rows[op] / (kernel_ms[op] * 1e-3) / 1e9
            per_kernel[op].update({"dram_traffic_gbs": dram, "dram_traffic_frac": dram / peak})
    top = max(kernel_ms, key=kernel_ms.get)
    roofline = {"bound": "hbm", "kernel": {"get": "k_get", "set": "k_set_claim (+ k_set_resolve, idle without duplicates)",
                                           "remove": "k_find<remove>"}[top],
                "achieved": per_kernel[top]["achieved_gbs"], "peak": peak, "unit": "GB/s", "frac": per_kernel[top]["frac"],
                "traffic": TRAFFIC_BYTES_PER_OP.get(top, 0) * local_rows[top] * passes if TRAFFIC_BYTES_PER_OP.get(top) else None,
                "peak_source": peak_source, "launches_per_operation": passes,
                "random_request_ceiling_greq_s": ceiling_window,
                "random_request_ceiling_whole_table_greq_s": ceiling_whole,
                "table_passes": passes,
                "note": ("phase time includes routing and exchange when shards > 1" +
                         (", measured with the operations called one after the other (the timed steps pipeline them); "
                          if pipelined else "; ") if world > 1 else "") +
                        "DRAM answers a random access with a whole 128-byte line whatever the request size (ncu: 122.7 B "
                        "read per 8-byte request, unchanged by cudaLimitMaxL2FetchGranularity), so a probing kernel is "
                        "bound by lines touched per operation (~46 G lines/s = the HBM bandwidth), not by the bytes it "
                        "needs; a slot array beyond the 64 GiB the TLB covers is served in passes over windows "
                        "(table_passes), see kernels.*.dram_traffic_frac for the share of the HBM peak each kernel moves"}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        _, _, cpu_baseline = cpu_arm(steps=4, warmup=1, sample_keys_log2=CPU_SAMPLE_KEYS_LOG2,
                                     sample_batch_log2=CPU_SAMPLE_BATCH_LOG2, budget_s=25.0)

    extra = {}
    if rank == 0 and world == 1:
        table.close()
        del table, local, slots, batches, d0
        torch.cuda.empty_cache()
        if args.scaling == "strong" and not args.no_shard_point:
            extra["shard_point"] = shard_point(torch, device)
            torch.cuda.empty_cache()
        if not args.no_extras:
            import bench_configs
            extra["configs"] = bench_configs.run_all(torch, device, measured_peak_gbs()[0])

    if rank == 0:
        line = {
            "metric": "hashmap get/set Mops/s", "value": value, "unit": "Mops/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling,
            "vs_baseline": None, "dtype": "int64", "data": "synthetic", "config": workload_config(args, world),
            "roofline": roofline, "kernels": per_kernel, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": int(launches), "clocks": clocks, "checks": checks,
            "mean_probe_groups": probe_len, "host_enqueue_ms_per_step": host_enqueue_ms,
            "exchange_phases_ms": exchange_phases, **extra,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def hw_probe(args):
    """Random-request rates of this GPU: the physical ceiling the roofline discussion rests on.  For every footprint
    and request shape, G requests/s over a buffer of that size.  Run under `ncu --metrics dram__bytes_read.sum` (one
    small footprint, --probe-reps 1) the same launches give the DRAM bytes per request."""
    import ctypes
    import torch
    from doksparse_b200 import _lib as L
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    torch.zeros(1, device=device)
    limit = {"requested": args.l2_fetch_granularity}
    cudart = ctypes.CDLL("libcudart.so.12")
    if args.l2_fetch_granularity:
        limit["set_rc"] = cudart.cudaDeviceSetLimit(5, ctypes.c_size_t(args.l2_fetch_granularity))    # cudaLimitMaxL2FetchGranularity
    got = ctypes.c_size_t(0)
    cudart.cudaDeviceGetLimit(ctypes.byref(got), 5)
    limit["reads_back"] = got.value
    shapes = [(8, 1), (16, 1), (32, 1), (32, 2), (32, 4), (16, 4)]
    n = 1 << args.probe_requests_log2
    lib = L.lib()
    rows = []
    for mib in args.probe_mib:
        try:
            buf = torch.empty(mib << 20, device=device, dtype=torch.uint8)
        except torch.OutOfMemoryError:
            rows.append({"mib": mib, "error": "out of memory"})
            continue
        buf.fill_(1)
        row = {"mib": mib}
        for b, lanes in shapes:
            if args.probe_reps > 1:
                L.check(lib.dok_diag_random_requests(L.ptr(buf), buf.numel(), n, b, lanes, 1, None, L.stream_ptr(device)), "probe")
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for rep in range(args.probe_reps):
                L.check(lib.dok_diag_random_requests(L.ptr(buf), buf.numel(), n, b, lanes, 100 + rep * n, None,
                                                     L.stream_ptr(device)), "probe")
            t1.record()
            torch.cuda.synchronize()
            row[f"{b * lanes}B_by_{lanes}_lane{'s' if lanes > 1 else ''}" + ("_16B_each" if (b, lanes) == (16, 4) else "")] = \
                round(args.probe_reps * n / (t0.elapsed_time(t1) * 1e-3) / 1e9, 2)
        rows.append(row)
        del buf
        torch.cuda.empty_cache()
    print(json.dumps({"hw_probe": "G random requests per second", "requests_per_launch": n,
                      "l2_fetch_granularity_limit": limit, "rows": rows}))


def small_dok(args):
    """One launch each of the DOK-side and routing kernels on small inputs (tables of 0.27-0.54 GB: a few times L2)."""
    import torch
    from doksparse_b200 import SparseDOKTensor
    from doksparse_b200.sharded import CudaShardOps
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    g = torch.Generator(device=device).manual_seed(0)
    n_rows = n_cols = 1 << 15
    lin = torch.unique(torch.randint(0, n_rows * n_cols, (5 << 20,), generator=g, device=device))[: 1 << 22]
    np.random.seed(0)
    t = SparseDOKTensor((n_rows, n_cols), torch.stack([lin // n_cols, lin % n_cols]), torch.randn(lin.numel(), generator=g, device=device))
    i = torch.randint(0, n_rows, (1 << 22,), generator=g, device=device)
    j = torch.randint(0, n_cols, (1 << 22,), generator=g, device=device)
    out = {"nnz": int(lin.numel()), "n_buckets": t.storage().n_buckets}
    got = t[i, j]                                                    # k_get over SelKeys
    t[i, j] = 1.0                                                    # k_set_claim over SelKeys (with its rehash)
    coo = t.to_sparse_coo()                                          # k_compact_count / k_compact_scatter
    block = torch.randn(4096, 4096, generator=g, device=device) * (torch.rand(4096, 4096, generator=g, device=device) < 0.01)
    d = SparseDOKTensor.from_dense(block)                            # k_dense_count / k_dense_insert
    ops = CudaShardOps(device, 1024, fixed_parameters(), 2.0, 0.75)
    idx = torch.arange(1 << 24, device=device)
    keys, values = mix62_torch(idx)[:, None].contiguous(), value_of_index(idx, torch).contiguous()
    gk, gv, dest, counts = ops.partition(keys, values, 8)           # k_part_count / scan / k_part_scatter<staged>
    ops.unpermute(gv, None, dest)                                    # k_unpermute
    torch.cuda.synchronize()
    out.update({"getitem_sum": float(got.sum()), "coo_nnz": int(coo._nnz()), "from_dense_nnz": d._nnz(),
                "partition_counts": counts[0].tolist()})
    print(json.dumps({"small_dok": out}))


def main():
    args = parse_args()
    if args.small_dok:
        small_dok(args)
    elif args.hw_probe:
        hw_probe(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_candidate(args)


if __name__ == "__main__":
    main()
