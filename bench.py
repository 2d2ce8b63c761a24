#!/usr/bin/env python
"""bench.py -- 4 KiB-page IOPS / GB/s through the GPU page cache (skewed array scan).

Workload (the multi-GPU skewed array scan configuration): a 64 GiB backing store of
splitmix64(seed ^ i) elements, sharded by contiguous 4 KiB-page range over the N ranks, one
16 GiB page cache and 128 x 1024 NVMe queue pairs per GPU; every step each GPU performs
2^26 element reads (2^20 reader lanes x 64) whose page popularity is Zipf(0.99) over its
shard (seeded rank permutation) with a uniform offset in the page.  One step = one cold run, as
every run of the reference's benchmarks is: the cache is emptied (a 30 us kernel, inside the timed
region) and one fused launch (emulated NVMe controller blocks + reader blocks) performs the reads.  Output per rank: the wrapping 64-bit sum,
verified on the device against the store's definition and reduced over ranks.

    python bench.py --gpus N --steps K --warmup W            the CUDA path
    python bench.py --impl reference ...                     the CPU restatement on host cores

One JSON line on rank 0.  `value` is whole-job 4 KiB page reads per second with the access lists
resident in HBM; `e2e` repeats it with the lists copied from pinned host memory and the result
read back inside the timed region.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

STORE_SEED, PERM_SEED, ACCESS_SEED = 0x5EED, 17, 23
PAGE = 4096
EPP = PAGE // 8


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="bam", choices=["bam", "reference"])
    ap.add_argument("--store-gib", type=float, default=64.0, help="total backing store over all ranks")
    ap.add_argument("--cache-gib", type=float, default=16.0, help="page cache per GPU")
    ap.add_argument("--lanes", type=int, default=1 << 20)
    ap.add_argument("--reqs", type=int, default=64)
    ap.add_argument("--queues", type=int, default=128)
    ap.add_argument("--depth", type=int, default=1024)
    ap.add_argument("--ctrl-blocks", type=int, default=0)
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--workload", default="zipf", choices=["zipf", "bfs", "cc", "sssp", "pagerank", "block", "array", "hit"],
                    help="zipf = the headline skewed array scan; bfs / cc = graph traversals through bam::array; "
                         "block = raw 4 KiB random reads (queue count x depth sweep); array = uniform random reads, 1 queue pair; "
                         "hit = element reads that all hit a small warm cache (the case profiled for the hit path)")
    ap.add_argument("--reqs-log2", type=int, default=24, help="block: log2 of the requests per sweep point")
    ap.add_argument("--scale", type=int, default=0, help="R-MAT scale for bfs (default 24) / cc (default 26)")
    ap.add_argument("--graph-cache-gib", type=float, default=0.0, help="page cache per GPU of the graph steps (default: 4 for BFS, 8 for CC)")
    ap.add_argument("--graph-steps", type=int, default=5, help="timed traversals per graph in the default run (BFS: twice as many)")
    ap.add_argument("--no-graphs", action="store_true", help="default run: skip the BFS and CC parts")
    ap.add_argument("--no-extras", action="store_true",
                    help="default run: skip the single-queue array read and the block-level sweep (the two other configurations)")
    ap.add_argument("--graphs-last", action="store_true", help="default run: BFS and CC after the array scan instead of before it")
    ap.add_argument("--cpu-sample-lanes", type=int, default=1 << 12)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ctrls", type=int, default=1, help="zipf: controllers behind each GPU's cache")
    ap.add_argument("--dist", default="stripe", choices=["stripe", "replicate"],
                    help="zipf with --ctrls > 1: how the array's pages are laid out over the controllers")
    ap.add_argument("--sys-scope", action="store_true",
                    help="synchronise doorbells and completions at system scope (default: device scope, enough when the controller runs on the same GPU)")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi during the timed region."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if not self.proc:
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
                for n, v in zip(names, r[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                pass
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def measured_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return None


def fill_touched_pages(orc, store, first_elem, idx):
    pages = np.unique(idx // np.uint64(EPP))
    orc.fill_pages(store, STORE_SEED, first_elem, pages, EPP)
    return len(pages)


def cpu_reference_step(orc, n_local_pages, first_page, cache_pages, queues, depth, lanes, reqs, access_seed,
                       workers, ctrl_threads, store, cdf):
    """One bounded sample of the workload through the CPU restatement of the reference's queue
    and cache protocol.  Returns (RefResult, seconds spent in the timed access loop)."""
    idx = orc.zipf_indices(cdf, n_local_pages, EPP, PERM_SEED, access_seed, 0, lanes, reqs)
    fill_touched_pages(orc, store, first_page * EPP, idx)
    r = orc.ref_array_read(store, PAGE, cache_pages, queues, depth, 512, workers, ctrl_threads, idx=idx,
                           lane_end=lanes, reqs_per_lane=reqs)
    want = orc.indexed_checksum(STORE_SEED, first_page * EPP, idx)
    if r.checksum != want:
        raise RuntimeError("CPU restatement checksum mismatch")
    return r


def cpu_reference_code_step(orc, n_local_pages, first_page, cache_slots, n_qps, depth, lanes, reqs, access_seed, workers, store, cdf):
    """The same bounded sample through the REFERENCE'S OWN cache and queue code (include/page_cache.h and
    include/nvm_parallel_queue.h compiled for host threads, oracle/_ref/libref_cache.so), each queue pair served
    by one controller thread of the oracle.  Returns (stats, seconds)."""
    idx = orc.zipf_indices(cdf, n_local_pages, EPP, PERM_SEED, access_seed, 0, lanes, reqs)
    fill_touched_pages(orc, store, first_page * EPP, idx)
    world = orc.RefCacheWorld(store, n_slots=cache_slots, n_qps=n_qps, qs=min(depth, 64))
    try:
        t0 = time.time()
        st = world.read(idx, n_threads=workers, timeout_ms=600000)
        dt = time.time() - t0
    finally:
        world.close()
    if st.checksum != orc.indexed_checksum(STORE_SEED, first_page * EPP, idx):
        raise RuntimeError("reference code checksum mismatch")
    return st, dt


def reference_code_available(orc):
    try:
        return orc.ref_cache() is not None
    except Exception:
        return False


def run_reference(args, rank, world):
    """--impl reference: the reference's own algorithm for this path restated for host threads
    (the reference cannot be built to run here: its host library needs /dev/libnvm* and its
    device headers do not compile for a host).  Rank 0 alone runs it."""
    if rank != 0:
        return
    from oracle import pyoracle as orc
    cores = os.cpu_count() or 1
    ctrl_threads = max(1, cores // 8)
    workers = max(1, cores - ctrl_threads)
    total_pages = int(args.store_gib * (1 << 30)) // PAGE
    n_local = total_pages // world
    cache_pages = int(args.cache_gib * (1 << 30)) // PAGE
    cdf = orc.zipf_cdf(n_local)
    store = np.empty(n_local * EPP, dtype=np.uint64)        # virtual; only touched pages are filled
    lanes = args.cpu_sample_lanes
    # shrink the in-memory cache of the sample to what the sample can touch
    cache_slots = min(cache_pages, lanes * args.reqs)
    times, ios, acc, misses = [], 0, 0, 0
    use_ref_code = reference_code_available(orc)
    for s in range(args.warmup + args.steps):
        if use_ref_code:
            st, dt = cpu_reference_code_step(orc, n_local, 0, cache_slots, ctrl_threads, args.depth, lanes, args.reqs,
                                             ACCESS_SEED + 1000 + s, workers, store, cdf)
            if s >= args.warmup:
                times.append(dt); ios += st.read_ios; acc += st.accesses; misses += st.misses
        else:
            r = cpu_reference_step(orc, n_local, 0, cache_slots, min(args.queues, 128), args.depth, lanes, args.reqs,
                                   ACCESS_SEED + 1000 + s, workers, ctrl_threads, store, cdf)
            if s >= args.warmup:
                times.append(r.seconds); ios += r.read_ios; acc += r.accesses; misses += r.misses
    t = sum(times)
    value = ios / t
    qps_used = ctrl_threads if use_ref_code else min(args.queues, 128)
    depth_used = min(args.depth, 64) if use_ref_code else args.depth
    sample = (f"{lanes} lanes x {args.reqs} reads per step of the same Zipf(0.99) stream over one {n_local}-page shard, "
              f"cold cache of {cache_slots} slots each step, {workers} reader threads + {ctrl_threads} controller threads; "
              + ("the reference's own page cache and queue code compiled for host threads (oracle/_ref), "
                 f"{qps_used} queue pairs of depth {depth_used}" if use_ref_code
                 else "CPU restatement of the reference's protocol"))
    # the config says what THIS arm ran: a bounded sample of the workload, on rank 0's host cores only
    cfg = workload_config(args, world)
    cfg.update({"sample_of": cfg["workload"] + f": {args.lanes * args.reqs} reads per GPU per step, {args.queues} x {args.depth} "
                             f"queues and a {args.cache_gib} GiB cache per GPU, {world} shard(s)",
                "workload": "bounded CPU sample of the multi-GPU skewed array scan (one shard, host threads)",
                "shards_run": 1, "reads_per_gpu_per_step": lanes * args.reqs, "queues_per_gpu": qps_used,
                "queue_depth": depth_used, "cache_gib_per_gpu": cache_slots * PAGE / (1 << 30), "cache_slots": cache_slots,
                "reader_threads": workers, "controller_threads": ctrl_threads})
    line = {
        "impl": "reference", "metric": "4KB-page IOPS via page cache", "value": value, "unit": "IOPS",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t / max(1, args.steps),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u64", "data": "synthetic",
        "config": cfg,
        "gb_per_s": value * PAGE / 1e9, "accesses_per_s": acc / t, "hit_rate": 1.0 - misses / max(1, acc),
        "cpu_baseline": {"value": value, "unit": "IOPS", "cores": workers + ctrl_threads, "kind": "reference" if use_ref_code else "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "IOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "one host runs one shard's sample whatever --gpus says: compare it with the per-GPU figures of the CUDA arm; "
                "a cold sample of this length has a lower hit rate than the full step, so compare accesses_per_s as well as IOPS",
    }
    print(json.dumps(line), flush=True)


def workload_config(args, world):
    return {"workload": "multi-GPU skewed array scan (Zipf 0.99 page popularity) through the page cache",
            "store_gib_total": args.store_gib, "shards": world, "cache_gib_per_gpu": args.cache_gib,
            "page_bytes": PAGE, "queues_per_gpu": args.queues, "queue_depth": args.depth,
            "reads_per_gpu_per_step": args.lanes * args.reqs, "zipf_s": 0.99, "cache_at_step_start": "empty",
            "queue_scope": "system" if args.sys_scope else "device",
            "controllers_per_gpu": max(1, args.ctrls), "distribution": args.dist if args.ctrls > 1 else "single controller",
            "l2": "inputs (cache + access lists) far larger than L2; no explicit flush"}


def verify_bfs(off, cols, lv, src):
    """Size-independent BFS properties, checked on the device against a plain copy of the CSR:
    source at level 0, every edge spans at most one level, neighbours of reached vertices are
    reached, every reached vertex but the source has a neighbour one level closer."""
    import torch
    n = off.numel() - 1
    lv = lv.to(torch.int64) & 0xFFFFFFFF
    srcs = torch.repeat_interleave(torch.arange(n, device=off.device), off[1:] - off[:-1])
    lu, lw = lv[srcs], lv[cols]
    inf = 0xFFFFFFFF
    reach = lu != inf
    ok = bool(lv[src] == 0) and bool(((lu[reach] - lw[reach]).abs() <= 1).all()) and bool((lw[reach] != inf).all())
    has_parent = torch.zeros(n, dtype=torch.bool, device=off.device)
    has_parent[srcs[(lw == lu - 1) & reach]] = True
    return ok and bool(has_parent[(lv != inf) & (lv != 0)].all())


def cc_fixed_point(off, cols):
    """Min-vertex component labels computed independently of the library: label propagation with plain
    tensor operations on the copy of the CSR in GPU memory (every vertex takes the minimum over its
    neighbours, then one pointer jump), iterated to the fixed point.  Edge sources are recovered in
    chunks so that the working set stays a fraction of the edge list."""
    import torch
    n, dev = off.numel() - 1, off.device
    lab = torch.arange(n, dtype=torch.int64, device=dev)
    chunk = 1 << 22                                     # vertices per chunk
    while True:
        new = lab.clone()
        for v0 in range(0, n, chunk):
            v1 = min(n, v0 + chunk)
            e0, e1 = int(off[v0].item()), int(off[v1].item())
            if e1 == e0:
                continue
            srcs = torch.repeat_interleave(torch.arange(v0, v1, device=dev), off[v0 + 1:v1 + 1] - off[v0:v1])
            nb = cols[e0:e1]
            new.scatter_reduce_(0, srcs, lab[nb], reduce="amin", include_self=True)
            new.scatter_reduce_(0, nb, lab[srcs], reduce="amin", include_self=True)
            del srcs
        new = torch.minimum(new, new[new])
        if bool((new == lab).all()):
            return lab
        lab = new


def verify_cc(off, cols, lab):
    """Exact: the labels equal the independently computed min-vertex labels (cc_fixed_point) bit for bit."""
    return bool((cc_fixed_point(off, cols) == lab).all())


def graph_cpu_baselines(args, keep, cc_cache_pages):
    """The same traversals through the CPU restatement of the reference's cache and queues on all host
    cores, cold cache of the same size: BFS on the very store image the GPU run used (result compared
    with the GPU's levels), CC on that same scale-24 graph as a bounded sample.  Returns (bfs, cc)."""
    from oracle import pyoracle as orc
    cores = os.cpu_count() or 1
    ctrl_threads = max(1, cores // 8)
    workers = max(1, cores - ctrl_threads)
    out = []
    for kind in (0, 1):
        try:
            vres, sc, it, r = orc.ref_graph_run(keep["store"], keep["n"], keep["off_bytes"], kind, keep["src"] if kind == 0 else 0,
                                                keep["bfs_cache_pages"] if kind == 0 else cc_cache_pages,
                                                min(args.queues, 128), args.depth, workers, ctrl_threads)
            b = {"value": sc / r.seconds / 1e9, "unit": "GTEPS", "cores": workers + ctrl_threads, "kind": "port",
                 "seconds": r.seconds, "read_ios": r.read_ios}
            if kind == 0:
                b["sample"] = "the whole traversal on the same backing store, cold cache of the same size"
                b["matches_gpu_result"] = bool((vres.view(np.int32) == keep["levels"]).all())
            else:
                b["sample"] = (f"CC over the R-MAT scale {keep['scale']} graph of the BFS step (a bounded sample), "
                               "cold cache of the same size as the GPU's")
        except Exception as e:
            b = {"value": None, "unit": "GTEPS", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
        out.append(b)
    return out


def measure_graph(kind, args, rank, world, dev_index, steps, warmup, link_agg):
    """BFS (R-MAT scale 24, 4 GiB cache) or CC (scale 26, 8 GiB cache) over a CSR graph whose offsets
    and edges are read only through bam::array; one step = one whole traversal from a cold cache.
    With N > 1 ranks the graph is sharded by vertex range (each rank's rows in its own backing
    store, cache and queues), labels are replicated and the frontier / changed labels are exchanged
    by NCCL all-gather after every level (compaction and apply kernels around the collective).
    Returns the result object on rank 0 (None elsewhere); torch.distributed must be initialised
    when world > 1.  `link_agg`: pinned-copy GB/s of all ranks at once (the host-link roofline)."""
    import torch
    import torch.distributed as dist
    import bam_b200
    dev = torch.device("cuda", dev_index)
    bfs = kind == "bfs"
    scale = args.scale or (24 if bfs else 26)
    cache_gib = args.graph_cache_gib or (4.0 if bfs else 8.0)
    t0 = time.time()
    off, cols = bam_b200.build_rmat_csr(1, scale, 16, device=dev)
    n, m = off.numel() - 1, cols.numel()
    src = int(torch.argmax(off[1:] - off[:-1]).item())          # highest degree, lowest id on ties
    kw = dict(cache_pages=int(cache_gib * (1 << 30)) // PAGE, cuda_device=dev_index, queue_depth=args.depth,
              num_queues=args.queues, ctrl_blocks=args.ctrl_blocks)
    gr = bam_b200.DistCsrGraph(off, cols, rank, world, **kw) if world > 1 else bam_b200.CsrGraph(off, cols, **kw)
    loc = gr.local if world > 1 else gr
    setup_s = time.time() - t0
    times, times_e2e, scanned, iters, ios = [], [], 0, 0, []
    out = None
    # the end-to-end span of a step ends when the labels are in pinned host memory (the graph itself always comes
    # from pinned host memory, page by page, through the controller)
    h_out = torch.empty(n, dtype=torch.int32 if bfs else torch.int64).pin_memory()
    for s in range(warmup + steps):
        loc.cache.invalidate()
        loc.cache.stats(reset=True)
        a, b, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a.record()
        out, iters, scanned = gr.bfs(src) if bfs else gr.cc()
        b.record()
        h_out.copy_(out, non_blocking=True)
        c.record()
        torch.cuda.synchronize()
        loc.ctrl.check_status()
        if s >= warmup:
            times.append(a.elapsed_time(b)); times_e2e.append(a.elapsed_time(c)); ios.append(loc.cache.stats()["read_ios"])
    prof = loc.ctrl.profile(reset=True)                       # zeros unless the library was built with -DBAM_PROFILE
    t_verify = time.time()
    ok = verify_bfs(off, cols, out, src) if bfs else verify_cc(off, cols, out)
    ok = ok and loc.cache.audit() == 0
    same = 1.0
    if world > 1:                                                # every replica must hold the same bits
        ref = out.clone()
        dist.broadcast(ref, 0)
        same = float(bool((ref == out).all()))
    verify_s = time.time() - t_verify
    red = torch.tensor([float(scanned), float(np.mean(ios)), float(ok), same], dtype=torch.float64, device=dev)
    step_ms = torch.tensor(times, dtype=torch.float64, device=dev)          # every step starts at a barrier: a step takes as long as its slowest rank
    e2e_ms = torch.tensor(times_e2e, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(step_ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(red, op=dist.ReduceOp.SUM)
    scanned_all, ios_all, n_ok, n_same = (float(x) for x in red.tolist())
    step_ms = step_ms.tolist()
    res = None
    if rank == 0:
        t = float(np.mean(step_ms)) * 1e-3
        t_med = float(np.median(step_ms)) * 1e-3
        link = ios_all * PAGE / t_med / 1e9
        res = {"gteps": scanned_all / t / 1e9, "ms": t * 1e3, "gteps_median_step": scanned_all / t_med / 1e9, "ms_median_step": t_med * 1e3,
               "ms_steps": [round(float(x), 2) for x in step_ms],
               ("levels" if bfs else "sweeps"): iters,
               "steps": steps, "warmup": warmup,
               "graph": f"R-MAT scale {scale}, edge factor 16 (a,b,c = .57,.19,.19), undirected, de-duplicated",
               "vertices": n, "directed_edges": m, "cache_gib_per_gpu": cache_gib, "source": src if bfs else None,
               "sharding": "vertex range, edge balanced" if world > 1 else "none",
               "edges_scanned": scanned_all, "read_ios": ios_all,
               "roofline": {"bound": "host_link", "achieved": link, "peak": link_agg, "unit": "GB/s",
                            "frac": link / link_agg if link_agg else None,
                            "kernel": "bam_fused<BfsLevelWork>" if bfs else "bam_fused<CcSweepWork>",
                            "note": "cold traversal, median step (the host uplink is shared with other tenants' GPUs and single steps "
                                    "are at times several times slower; every step is listed in ms_steps): read_ios x 4096 B cross "
                                    "the host link; peak = pinned-memory H2D copy "
                                    "measured in this run on all ranks at once"},
               "verified": bool(n_ok == world and n_same == world),
               "verified_how": ("levels pinned by the BFS certificate on the CSR in GPU memory" if bfs else
                                "labels equal an independent min-label fixed point computed with tensor operations on the CSR in GPU memory")
                               + ("; every rank's replica equal to rank 0's bit for bit" if world > 1 else ""),
               "e2e": {"value": scanned_all / (float(e2e_ms.mean().item()) * 1e-3) / 1e9, "unit": "GTEPS",
                       "ms": float(e2e_ms.mean().item()), "ms_median_step": float(e2e_ms.median().item()),
                       "h2d_bytes_per_step": int(ios_all * PAGE), "d2h_bytes_per_step": int(h_out.numel() * h_out.element_size() * world),
                       "note": "the traversal call with the graph in pinned host memory (every page it reads crosses the host link "
                               "inside the timed span) plus the copy of the labels to pinned host memory"},
               "gpu_launches": (iters * (3 if world > 1 else 1)) * (steps + warmup), "setup_s": setup_s, "verify_s": verify_s}
        if world > 1 and not bfs:
            res["dense_exchange_sweeps"] = getattr(gr, "cc_dense_sweeps", None)
        if any(prof):
            res["protocol_counters"] = protocol_counters(prof)
    keep = None
    if bfs and world == 1 and not args.no_cpu_baseline:
        # what the CPU baselines need later (they run after every GPU measurement): the store image, the
        # GPU's levels to compare with, and the cache geometry
        keep = {"store": loc.ctrl.store_numpy().copy(), "n": n, "off_bytes": loc.off_bytes, "scale": scale, "src": src,
                "levels": out.cpu().numpy().copy(), "bfs_cache_pages": kw["cache_pages"]}
    gr.close()
    del off, cols, out
    torch.cuda.empty_cache()
    return res, keep


def run_graph(args, rank, world, local_rank):
    """--workload bfs | cc: the traversal alone, one JSON line."""
    import torch
    import torch.distributed as dist
    import bam_b200
    dev_index, placement = bam_b200.place_rank(world, local_rank, f"{os.environ.get('MASTER_PORT', '0')}_{os.getppid()}")
    torch.cuda.set_device(dev_index)
    dev = torch.device("cuda", dev_index)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    bam_b200.bind_to_gpu_numa(dev_index)
    bfs = args.workload == "bfs"
    _, link_agg = measure_link_rate(torch, dist, dev, world, 3)
    sampler = ClockSampler(dev_index)
    if rank == 0:
        sampler.start()
    res, keep = measure_graph(args.workload, args, rank, world, dev_index, args.steps, args.warmup, link_agg)
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        if keep is not None:
            res["cpu_baseline"] = graph_cpu_baselines(args, keep, 0)[0]
        line = {"metric": "BFS GTEPS through bam::array" if bfs else "CC GTEPS through bam::array",
                "value": res["gteps"], "unit": "GTEPS", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": res["ms"], "ms_best_step_rank0": min(res["ms_steps"]), "ms_steps_rank0": res["ms_steps"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "u64", "data": "synthetic",
                "config": {"workload": f"{'BFS' if bfs else 'CC'} over {res['graph']}; u64 offsets and edges read through the "
                                       "page cache, cold cache at the start of every traversal",
                           "queues": args.queues, "queue_depth": args.depth, "placement": placement,
                           "l2": "graph (GiB) far larger than L2; no explicit flush"},
                "clocks": clocks}
        line.update(res)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def measure_link_rate(torch, dist, dev, world, reps):
    """Pinned-memory H2D copy rate of this rank while every rank copies: (per-GPU mean, aggregate) in GB/s."""
    stream = torch.cuda.current_stream()
    pin = torch.empty(1 << 30, dtype=torch.uint8).pin_memory()
    dbuf = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
    best = 0.0
    for _ in range(reps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream); dbuf.copy_(pin, non_blocking=True); b.record(stream); stream.synchronize()
        best = max(best, (1 << 30) / (a.elapsed_time(b) * 1e-3) / 1e9)
    del pin, dbuf
    link = torch.tensor([best], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(link, op=dist.ReduceOp.SUM)
    return float(link.item()) / world, float(link.item())


def verify_sssp(off, cols, wts, dist, src):
    """A certificate of shortest-path distances with positive weights, checked on the device:
    dist[src] == 0; no edge out of a reached vertex can shorten its head (so heads of reached
    vertices are reached); every reached vertex but the source has an edge that it is tight on."""
    import torch
    n = off.numel() - 1
    inf = 0xFFFFFFFF
    d = dist.to(torch.int64) & inf
    srcs = torch.repeat_interleave(torch.arange(n, device=off.device), off[1:] - off[:-1])
    du, dv, w = d[srcs], d[cols], wts.to(torch.int64)
    reach = du != inf
    ok = bool(d[src] == 0) and bool((dv[reach] <= du[reach] + w[reach]).all())
    tight = torch.zeros(n, dtype=torch.bool, device=off.device)
    tight[cols[reach & (dv == du + w)]] = True
    need = (d != inf)
    need[src] = False
    return ok and bool(tight[need].all())


def verify_pagerank(off, cols, value, sweeps, alpha=(85, 100), frac_bits=40, max_iters=100):
    """The same fixed-point sweeps recomputed with plain tensor operations on a copy of the CSR in
    GPU memory (integer adds commute, so the result must be identical bit for bit)."""
    import torch
    n = off.numel() - 1
    dev = off.device
    num, den = alpha
    ratio = lambda x: x // den * num + (x % den) * num // den  # noqa: E731
    one = 1 << frac_bits
    tol = one // 1000
    deg = off[1:] - off[:-1]
    degc = deg.clamp(min=1)
    srcs = torch.repeat_interleave(torch.arange(n, device=dev), deg)
    base = one - (one // den * num + (one % den) * num // den)
    val = torch.full((n,), base, dtype=torch.int64, device=dev)
    delta = torch.where(deg > 0, torch.full((n,), ratio(base), dtype=torch.int64, device=dev) // degc, torch.zeros_like(val))
    res = torch.zeros(n, dtype=torch.int64, device=dev)
    label = torch.ones(n, dtype=torch.bool, device=dev)
    it = 0
    while it < max_iters:
        res.index_add_(0, cols, torch.where(label[srcs], delta[srcs], torch.zeros((), dtype=torch.int64, device=dev)))
        it += 1
        label = res > tol
        if not bool(label.any()):
            break
        val = torch.where(label, val + res, val)
        delta = torch.where(label, torch.where(deg > 0, ratio(res) // degc, torch.zeros_like(res)), delta)
        res = torch.where(label, torch.zeros_like(res), res)
    return it == sweeps and bool((val == value).all())


def run_rank(args):
    """SSSP (label-correcting, u32 weights in a third array) or fixed-point PageRank over an R-MAT
    graph read only through bam::array; one step = one whole run from a cold cache; 1 GPU."""
    import torch
    import bam_b200
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    sssp = args.workload == "sssp"
    scale = args.scale or 24
    cache_gib = args.cache_gib if args.cache_gib != 16.0 else 4.0
    t0 = time.time()
    off, cols = bam_b200.build_rmat_csr(1, scale, 16, device=dev)
    n, m = off.numel() - 1, cols.numel()
    src = int(torch.argmax(off[1:] - off[:-1]).item())
    wts = None
    if sssp:
        # bam_edge_weight(seed, j) = 1 + (splitmix64(seed ^ j) >> 58), evaluated with tensor operations
        x = (torch.arange(m, dtype=torch.int64, device=dev) ^ 101) + (-7046029254386353131)
        z = (x ^ ((x >> 30) & ((1 << 34) - 1))) * (-4658895280553007687)
        z = (z ^ ((z >> 27) & ((1 << 37) - 1))) * (-7723592293110705685)
        z = z ^ ((z >> 31) & ((1 << 33) - 1))
        wts = (((z >> 58) & 63) + 1).to(torch.int32)
    gr = bam_b200.CsrGraph(off, cols, cache_pages=int(cache_gib * (1 << 30)) // PAGE, queue_depth=args.depth,
                           num_queues=args.queues, ctrl_blocks=args.ctrl_blocks, weights=wts)
    setup_s = time.time() - t0
    times, ios, out, iters, scanned = [], [], None, 0, 0
    sampler = ClockSampler(0)
    for s in range(args.warmup + args.steps):
        if s == args.warmup:
            sampler.start()
        gr.cache.invalidate()
        gr.cache.stats(reset=True)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        out, iters, scanned = gr.sssp(src) if sssp else gr.pagerank()
        b.record()
        torch.cuda.synchronize()
        gr.ctrl.check_status()
        if s >= args.warmup:
            times.append(a.elapsed_time(b)); ios.append(gr.cache.stats()["read_ios"])
    clocks = sampler.stop()
    ok = (verify_sssp(off, cols, wts, out, src) if sssp else verify_pagerank(off, cols, out, iters)) and gr.cache.audit() == 0
    t = float(np.mean(times)) * 1e-3
    line = {"metric": ("SSSP" if sssp else "PageRank") + " GTEPS through bam::array", "value": scanned / t / 1e9, "unit": "GTEPS",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "u32" if sssp else "u64 fixed point (40 fraction bits)",
            "data": "synthetic",
            "config": {"workload": ("SSSP, u32 weights 1..64 in a third array" if sssp else "push-based delta PageRank, alpha 0.85, "
                                    "tolerance 0.001, at most 100 sweeps") + f" over R-MAT scale {scale} edge factor 16, u64 offsets "
                       "and edges read through the page cache, cold cache at the start of every run",
                       "vertices": n, "directed_edges": m, "cache_gib_per_gpu": cache_gib, "queues": args.queues,
                       "queue_depth": args.depth, "source": src, "l2": "graph (GiB) far larger than L2; no explicit flush"},
            "sweeps": iters, "edges_scanned_per_step": scanned, "read_ios_per_step": float(np.mean(ios)),
            "link_gb_per_s": float(np.mean(ios)) * PAGE / t / 1e9, "verified": bool(ok), "gpu_launches": (iters + (0 if sssp else 1)) * args.steps,
            "clocks": clocks, "setup_s": setup_s}
    if not args.no_cpu_baseline:
        try:
            from oracle import pyoracle as orc
            cs = min(scale, 20)                                   # a bounded sample: the same generator at a smaller scale
            o, c = orc.rmat_csr(1, cs, 16)
            t1 = time.time()
            if sssp:
                orc.sssp(o, c, orc.edge_weights(101, len(c)), orc.max_degree_vertex(o))
                sc = len(c)
            else:
                _, _, sc = orc.pagerank(o, c)
            dt = time.time() - t1
            line["cpu_baseline"] = {"value": sc / dt / 1e9, "unit": "GTEPS", "cores": 1, "kind": "port",
                                    "sample": f"the result oracle ({'Dijkstra' if sssp else 'sequential sweeps'}) on the same generator "
                                              f"at scale {cs}, graph in host memory"}
        except Exception as e:
            line["cpu_baseline"] = {"value": None, "unit": "GTEPS", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
    print(json.dumps(line), flush=True)
    gr.close()


def run_block(args):
    print(json.dumps(measure_block(args)), flush=True)


def run_array(args):
    print(json.dumps(measure_array(args)), flush=True)


def protocol_counters(prof):
    """The 32 counters of a -DBAM_PROFILE build of the library (BAM_B200_LIB=...), per command / batch: where a
    command's life goes, in SM cycles, summed over everything the controller has run since they were last reset."""
    cmds, batches = max(1, prof[0]), max(1, prof[16])
    return {
        "commands": prof[0], "sq_turn_wait_cycles_per_cmd": prof[1] / cmds, "cid_cycles_per_cmd": prof[2] / cmds,
        "publish_cycles_per_cmd": prof[3] / cmds, "completion_wait_cycles_per_cmd": prof[4] / cmds,
        "reaps": prof[5], "cycles_per_reap": prof[6] / max(1, prof[5]), "entries_per_reap": prof[7] / max(1, prof[5]),
        "doorbell_sweeps": prof[8], "entries_per_sweep": prof[9] / max(1, prof[8]),
        "cache_lost_inserts": prof[10], "cache_evictions": prof[11], "cache_free_claims": prof[12],
        "cache_sweep_probes_per_claim": prof[13] / max(1, prof[11] + prof[12]),
        "ctrl_batches": prof[16], "ctrl_cmds_per_batch": prof[17] / batches, "ctrl_fetch_cycles_per_batch": prof[18] / batches,
        "ctrl_batch_cycles": prof[19] / batches, "ctrl_load_wait_cycles_per_cmd": prof[20] / max(1, prof[17]),
        "ctrl_load_and_store_cycles_per_cmd": prof[21] / max(1, prof[17]), "ctrl_post_cycles_per_cmd": prof[22] / max(1, prof[17]),
        "ctrl_idle_polls": prof[23], "ctrl_cycles_per_idle_poll": prof[24] / max(1, prof[23]),
        "note": "SM cycles at the clock printed by nvidia-smi; the counters add overhead of their own, the rates of this "
                "build are lower than the product build's"}


def measure_block(args):
    """Block-level random read throughput (the nvm-block-bench shape): 4 KiB reads at seeded random
    page-aligned offsets of a 16 GiB store, no cache reuse, swept over queue count x depth.  Every
    sweep point is verified: the wrapping sum of all words read must equal the sum recomputed from the
    store's definition, and a sample of the page CRC-32s is checked against the oracle's."""
    import torch
    import bam_b200
    from oracle import pyoracle as orc
    torch.cuda.set_device(0)
    store_gib = args.store_gib if args.store_gib != 64.0 else 16.0
    n_pages = int(store_gib * (1 << 30)) // PAGE
    n_reqs = 1 << args.reqs_log2
    points = []
    pages_d = torch.empty(n_reqs, dtype=torch.int64, device="cuda")
    want = torch.zeros(1, dtype=torch.int64, device="cuda")
    for nq in (1, 16, 64, 128):
        for depth in (64, 256, 1024):
            ctrl = bam_b200.Controller(n_pages * PAGE, 0, queue_depth=depth, num_queues=nq)
            ctrl.configure(ctrl_blocks=args.ctrl_blocks)
            ctrl.fill_store(STORE_SEED)
            g, _, th = ctrl.geometry()
            cache = bam_b200.PageCache(ctrl, PAGE, g * th)
            reqs = n_reqs if nq > 1 else min(n_reqs, 1 << 21)            # one queue is ~10x slower: bound the run
            out = torch.zeros(1, dtype=torch.int64, device="cuda")
            crc = torch.zeros(1 << 12, dtype=torch.int32, device="cuda")
            cache.block_read(1 << 12, req_seed=78, crc_out=crc)           # warm-up + CRC sample
            pg, wc = orc.block_requests(STORE_SEED, 78, n_pages, PAGE, 0, 1 << 12)
            ok = bool((crc.cpu().numpy().view(np.uint32) == wc).all())
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); cache.block_read(reqs, req_seed=79, sum_out=out); b.record(); torch.cuda.synchronize()
            ctrl.check_status()
            ms = a.elapsed_time(b)
            # expected sum: every word of every requested page, recomputed from the definition
            idx = torch.arange(reqs, dtype=torch.int64, device="cuda")
            bam_b200.gen_block_pages(pages_d[:reqs], reqs, 79, n_pages)
            want.zero_()
            bam_b200.page_sums(pages_d[:reqs], reqs, STORE_SEED, PAGE // 8, want)
            ok = ok and int(out.item()) == int(want.item())
            points.append({"queues": nq, "depth": depth, "requests": reqs, "iops": reqs / (ms * 1e-3),
                           "gb_per_s": reqs * PAGE / (ms * 1e-3) / 1e9, "verified": ok})
            cache.close(); ctrl.close()
    best = max(points, key=lambda p: p["iops"])
    line = {"metric": "4KB random-read IOPS (block level, no cache reuse)", "value": best["iops"], "unit": "IOPS",
            "n_gpus": 1, "steps": 1, "warmup": 1, "ms_per_step": None, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": "block-level 4 KiB random reads", "store_gib": store_gib, "requests_per_point": n_reqs,
                       "l2": "every request reads a different 4 KiB page of a store far larger than L2"},
            "sweep": points, "verified": all(p["verified"] for p in points), "gpu_launches": 2 * len(points)}
    return line


def measure_array(args):
    """Array random-read checksum (the nvm-array-bench shape): 2^27 u64 elements (1 GiB), 256 MiB cache,
    ONE queue pair of depth 1024, 2^20 reader lanes x 64 uniform indices; bit-exact wrapping sum."""
    import torch
    import bam_b200
    from oracle import pyoracle as orc
    torch.cuda.set_device(0)
    n_elems, lanes, reqs = 1 << 27, args.lanes, args.reqs
    ctrl = bam_b200.Controller(n_elems * 8, 0, queue_depth=args.depth, num_queues=1)
    ctrl.configure(ctrl_blocks=args.ctrl_blocks)
    ctrl.fill_store(STORE_SEED)
    cache = bam_b200.PageCache(ctrl, PAGE, 65536)
    arr = bam_b200.Array(cache, n_elems)
    out = torch.zeros(1, dtype=torch.int64, device="cuda")
    arr.read(1 << 12, reqs, out, access_seed=ACCESS_SEED + 1)          # warm-up launch
    torch.cuda.synchronize()
    times, sums = [], []
    for s in range(args.steps):
        cache.invalidate(); cache.stats(reset=True); out.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); arr.read(lanes, reqs, out, access_seed=ACCESS_SEED); b.record(); torch.cuda.synchronize()
        ctrl.check_status()
        times.append(a.elapsed_time(b)); sums.append(int(out.item()) & ((1 << 64) - 1))
    st = cache.stats()
    prof = ctrl.profile(reset=False)                                                 # zeros unless the library was built with -DBAM_PROFILE
    want = orc.array_checksum(STORE_SEED, n_elems, ACCESS_SEED, 0, lanes, reqs)       # the oracle needs no store
    t = float(np.mean(times)) * 1e-3
    line = {"metric": "array random-read through the page cache, 1 queue pair", "value": st["read_ios"] / t, "unit": "IOPS",
            "n_gpus": 1, "steps": args.steps, "warmup": 1, "ms_per_step": t * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "u64", "data": "synthetic",
            "config": {"workload": "array random-read checksum", "elements": n_elems, "cache_mib": 256, "queues": 1,
                       "queue_depth": args.depth, "lanes": lanes, "reads_per_lane": reqs,
                       "l2": "1 GiB store, 256 MiB cache: far larger than L2"},
            "checksum": f"{sums[-1]:#018x}", "verified": all(x == want for x in sums) and cache.audit() == 0,
            "elements_per_s": lanes * reqs / t, "gb_per_s": st["read_ios"] * PAGE / t / 1e9,
            "hit_rate": st["hits"] / max(1, st["accesses"]), "gpu_launches": args.steps}
    if any(prof):
        line["protocol_counters"] = protocol_counters(prof)
    arr.close(); cache.close(); ctrl.close()
    return line


def run_hit(args):
    """Element reads through array[] that all hit: a small warm cache (0.5 GiB resident, larger than L2),
    2^23 uniform random 8-byte reads, then 2^23 reads in the shape of the reference's cache benchmark
    (the 32 lanes of a warp read 32 consecutive elements per step, benchmarks/cache/main.cu:60-78).
    Launch order of bam_fused<...>: 1 page scan (fills the cache), 4 x random, 4 x sequential."""
    import torch
    import bam_b200
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    n_res = 1 << 17                                               # resident pages: 0.5 GiB
    n_reads = 1 << args.reqs_log2 if args.reqs_log2 != 24 else 1 << 23
    ctrl = bam_b200.Controller(n_res * PAGE, 0, queue_depth=args.depth, num_queues=args.queues)
    ctrl.configure(ctrl_blocks=args.ctrl_blocks)
    ctrl.fill_store(STORE_SEED)
    cache = bam_b200.PageCache(ctrl, PAGE, n_res * 2)
    arr = bam_b200.Array(cache, n_res * EPP)
    s = torch.zeros(1, dtype=torch.int64, device=dev)
    arr.page_scan(n_res, s, first_page=0)
    torch.cuda.synchronize(); ctrl.check_status(); cache.stats(reset=True)
    lanes, reqs = n_reads // 64, 64
    ridx = torch.empty(n_reads, dtype=torch.int64, device=dev)
    bam_b200.gen_uniform_indices(ridx, lanes, reqs, ACCESS_SEED + 77, n_res * EPP)
    seq = (torch.arange(n_reads // 2048, device=dev, dtype=torch.int64).view(-1, 1, 1) * 2048
           + torch.arange(64, device=dev, dtype=torch.int64).view(1, 1, 64) * 32
           + torch.arange(32, device=dev, dtype=torch.int64).view(1, 32, 1)).reshape(-1) % (n_res * EPP)
    res = {}
    for name, idx in (("random", ridx), ("sequential", seq)):
        want, got = torch.zeros(1, dtype=torch.int64, device=dev), torch.zeros(1, dtype=torch.int64, device=dev)
        bam_b200.direct_checksum(idx, n_reads, STORE_SEED, 0, want)
        times = []
        for _ in range(4):
            got.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); arr.read(lanes, reqs, got, idx=idx); b.record(); torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        ctrl.check_status()
        st = cache.stats(reset=True)
        t = float(np.mean(times[1:])) * 1e-3
        res[name] = {"reads_per_s": n_reads / t, "useful_gb_per_s": n_reads * 8 / t / 1e9, "ms": t * 1e3,
                     "misses": st["misses"], "verified": int(got.item()) == int(want.item())}
    # the reference's cache benchmark itself (sequential_access_warp, type ORIG): warp w reads whole pages through
    # array[], 32 consecutive elements per step, indices computed in the kernel
    ppw = 4
    want, got = torch.zeros(1, dtype=torch.int64, device=dev), torch.zeros(1, dtype=torch.int64, device=dev)
    arr.page_scan(n_res, want, first_page=0)
    times = []
    for _ in range(4):
        got.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); arr.pattern_read(1, n_res * EPP, got, n_warps=n_res // ppw, n_pages_per_warp=ppw, impl=1); b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    ctrl.check_status()
    st = cache.stats(reset=True)
    t = float(np.mean(times[1:])) * 1e-3
    res["cache_bench"] = {"reads_per_s": n_res * EPP / t, "useful_gb_per_s": n_res * PAGE / t / 1e9, "ms": t * 1e3,
                          "misses": st["misses"], "verified": int(got.item()) == int(want.item())}
    line = {"metric": "all-hit element reads through array[]", "value": res["random"]["reads_per_s"], "unit": "reads/s",
            "n_gpus": 1, "steps": 3, "warmup": 1, "ms_per_step": res["random"]["ms"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u64", "data": "synthetic",
            "config": {"workload": "warm all-hit element reads", "resident_pages": n_res, "reads": n_reads,
                       "l2": "0.5 GiB of resident pages + 64 MiB index list: larger than L2"},
            "random": res["random"], "sequential": res["sequential"], "cache_bench": res["cache_bench"],
            "audit": cache.audit(), "gpu_launches": 14}
    print(json.dumps(line), flush=True)
    arr.close(); cache.close(); ctrl.close()


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.workload in ("bfs", "cc"):
        run_graph(args, rank, world, local_rank)
        return
    if args.workload in ("sssp", "pagerank"):
        run_rank(args)
        return
    if args.workload in ("block", "array", "hit"):
        if rank == 0:
            {"block": run_block, "array": run_array, "hit": run_hit}[args.workload](args)
        return

    import torch
    import torch.distributed as dist
    import bam_b200
    from bam_b200 import _lib

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    # ranks are spread over distinct host uplinks first (matters when fewer ranks than GPUs run)
    dev_index, placement = bam_b200.place_rank(world, local_rank, f"{os.environ.get('MASTER_PORT', '0')}_{os.getppid()}")
    local_rank = dev_index                                  # from here on: the CUDA device of this rank
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    numa = bam_b200.bind_to_gpu_numa(local_rank)          # the pinned shard is placed next to its GPU
    total_pages = int(args.store_gib * (1 << 30)) // PAGE
    first_page, n_local = bam_b200.shard_pages(total_pages, world, rank)
    cache_pages = int(args.cache_gib * (1 << 30)) // PAGE
    if cache_pages > (1 << 24) - 2:
        raise SystemExit(f"--cache-gib {args.cache_gib}: {cache_pages} slots exceed the library's limit of 2^24 - 2 slots per cache")
    lanes, reqs = args.lanes, args.reqs
    n_acc = lanes * reqs

    # ---- the metric's second half: BFS and CC GTEPS through bam::array, on the same ranks ---------------
    graph_res = {}

    def graph_part():
        if args.no_graphs:
            return
        _, agg = measure_link_rate(torch, dist, dev, world, 3)
        gsteps, gwarm = max(1, min(args.steps, args.graph_steps)), 1
        bfs_res, keep = measure_graph("bfs", args, rank, world, local_rank, 2 * gsteps, gwarm, agg)
        cc_res, _ = measure_graph("cc", args, rank, world, local_rank, gsteps, gwarm, agg)
        graph_res["bfs"], graph_res["cc"], graph_res["keep"] = bfs_res, cc_res, keep

    def graph_part_guarded():
        # a failure of the traversal part must not cost the array-scan line; with several ranks it cannot be
        # contained (the other ranks would wait in a collective), so there it ends the run
        if world > 1:
            return graph_part()
        try:
            graph_part()
        except Exception as e:
            graph_res.clear()
            graph_res["error"] = f"{type(e).__name__}: {e}"

    if not args.graphs_last:
        graph_part_guarded()

    t0 = time.time()
    k_ctrls = max(1, args.ctrls)
    stripe = k_ctrls > 1 and args.dist == "stripe"
    if stripe:
        n_local -= n_local % k_ctrls                           # whole stripes
    per_ctrl_pages = n_local // k_ctrls if stripe else n_local
    ctrls = [bam_b200.Controller(per_ctrl_pages * PAGE, local_rank, queue_depth=args.depth, num_queues=args.queues)
             for _ in range(k_ctrls)]
    ctrl = ctrls[0]                                            # the first controller sets the launch geometry
    for k, c in enumerate(ctrls):
        c.configure(ctrl_blocks=args.ctrl_blocks, batch=args.batch)
        if args.sys_scope:
            c.set_scope(1)
        if stripe:
            c.fill_store_striped(STORE_SEED, k, k_ctrls, first_elem=first_page * EPP, page_bytes=PAGE)
        else:
            c.fill_store(STORE_SEED, first_elem=first_page * EPP)
    cache = bam_b200.PageCache(ctrls if k_ctrls > 1 else ctrl, PAGE, cache_pages)
    arr = bam_b200.Array(cache, n_local * EPP, dist=bam_b200.STRIPE if stripe else bam_b200.REPLICATE)
    cdf = bam_b200.zipf_cdf(n_local)
    d_cdf = torch.from_numpy(cdf.view(np.int64)).to(dev)
    torch.cuda.synchronize()
    setup_s = time.time() - t0

    n_steps = args.warmup + args.steps
    stream = torch.cuda.current_stream()
    sptr = stream.cuda_stream
    d_idx = [torch.empty(n_acc, dtype=torch.int64, device=dev) for _ in range(n_steps)]
    for s in range(n_steps):
        bam_b200.gen_zipf_indices(d_idx[s], lanes, reqs, ACCESS_SEED + 1000 * rank + s, d_cdf, n_local, EPP,
                                  PERM_SEED + rank, stream=sptr)
    sums = torch.zeros(n_steps, dtype=torch.int64, device=dev)
    want = torch.zeros(n_steps, dtype=torch.int64, device=dev)
    for s in range(n_steps):
        bam_b200.direct_checksum(d_idx[s], n_acc, STORE_SEED, first_page * EPP, want[s:s + 1], stream=sptr)
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def measure_link(reps):
        return measure_link_rate(torch, dist, dev, world, reps)

    # Pages the controller keeps in flight (16 per controller block) are sized to the bandwidth-delay product of
    # the link this rank really gets: GPUs that share a PCIe uplink see about half the bandwidth and twice the
    # latency under load, and flooding the shared switch with a full-rate window of 4 KiB reads costs throughput
    # (8 GPUs of one box: 48 blocks 45.2 M IOPS, 24 blocks 48.4 M).  48 blocks at 55 GB/s, in proportion below.
    ctrl_blocks = args.ctrl_blocks
    if ctrl_blocks == 0:
        link_before, _ = measure_link(2)
        ctrl_blocks = max(16, min(48, int(48.0 * link_before / 55.0 / 8.0 + 0.5) * 8))
        ctrl.configure(ctrl_blocks=ctrl_blocks)

    def run_step(s):
        cache.invalidate_async(stream=sptr)
        arr.read(lanes, reqs, sums[s:s + 1], idx=d_idx[s], stream=sptr)

    # ---- device-resident timing: value -------------------------------------------------------
    for s in range(args.warmup):
        run_step(s)
    ctrl.check_status()
    cache.stats(reset=True)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for k in range(args.steps):
        ev[k][0].record(stream)
        run_step(args.warmup + k)
        ev[k][1].record(stream)
    e1.record(stream)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ctrl.check_status()
    elapsed_ms = e0.elapsed_time(e1)
    kernel_ms = [a.elapsed_time(b) for a, b in ev]
    st = cache.stats(reset=True)
    ok = bool((sums == want).all().item())
    audit = cache.audit()

    # ---- end to end: access lists start in pinned host memory, result read back ----------------
    h_idx = torch.empty(n_acc, dtype=torch.int64).pin_memory()
    h_idx.copy_(d_idx[args.warmup])
    d_stage = torch.empty(n_acc, dtype=torch.int64, device=dev)
    e2e_sum = torch.zeros(1, dtype=torch.int64, device=dev)
    h_sum = torch.zeros(1, dtype=torch.int64).pin_memory()
    cache.stats(reset=True)
    barrier()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record(stream)
    for k in range(args.steps):
        d_stage.copy_(h_idx, non_blocking=True)
        e2e_sum.zero_()
        cache.invalidate_async(stream=sptr)
        arr.read(lanes, reqs, e2e_sum, idx=d_stage, stream=sptr)
        h_sum.copy_(e2e_sum, non_blocking=True)
        stream.synchronize()
    g1.record(stream)
    barrier()
    ctrl.check_status()
    e2e_ms = g0.elapsed_time(g1)
    st_e2e = cache.stats(reset=True)
    ok = ok and (int(h_sum.item()) == int(want[args.warmup].item()))

    # ---- host-link peak (pinned H2D copy) and warm hit-path pass (HBM roofline) ----------------
    # every rank copies at the same time: GPUs of one box share PCIe uplinks, so the per-GPU ceiling
    # under load is what the miss path of an N-rank run can be compared with
    _, link_agg = measure_link(5)
    link_gbs, hit = link_agg / world, None
    if rank == 0:
        # warm pass: scan pages that are resident (scan the same list twice, time the second)
        n_scan = min(cache_pages // 2, n_local)
        scan_sum = torch.zeros(1, dtype=torch.int64, device=dev)
        cache.invalidate()
        arr.page_scan(n_scan, scan_sum, first_page=0, stream=sptr)
        torch.cuda.synchronize()
        cache.stats(reset=True)
        times = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream); arr.page_scan(n_scan, scan_sum, first_page=0, stream=sptr); b.record(stream)
            stream.synchronize()
            times.append(a.elapsed_time(b))
        ctrl.check_status()
        sst = cache.stats(reset=True)
        hit = {"ms": float(np.mean(times[1:])), "pages": n_scan, "hits": sst["hits"], "misses": sst["misses"]}
        # random 8-byte reads that all hit: uniform indices over the pages the scan left resident
        n_rand = 1 << 26
        d_ridx = torch.empty(n_rand, dtype=torch.int64, device=dev)
        bam_b200.gen_uniform_indices(d_ridx, 1 << 20, 64, ACCESS_SEED + 77, n_scan * EPP, stream=sptr)
        rsum, rwant = torch.zeros(1, dtype=torch.int64, device=dev), torch.zeros(1, dtype=torch.int64, device=dev)
        bam_b200.direct_checksum(d_ridx, n_rand, STORE_SEED, first_page * EPP, rwant, stream=sptr)
        times = []
        for _ in range(4):
            rsum.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream); arr.read(1 << 20, 64, rsum, idx=d_ridx, stream=sptr); b.record(stream)
            stream.synchronize()
            times.append(a.elapsed_time(b))
        ctrl.check_status()
        rst = cache.stats(reset=True)
        hit_rand = {"ms": float(np.mean(times[1:])), "reads": n_rand, "misses": rst["misses"],
                    "ok": int(rsum.item()) == int(rwant.item())}
        # the reference's cache benchmark in `array[]` mode: the 32 lanes of a warp read 32 consecutive
        # elements per step, so one pin serves a whole warp (benchmarks/cache/main.cu:60-78)
        seq = (torch.arange(n_rand // 2048, device=dev, dtype=torch.int64).view(-1, 1, 1) * 2048
               + torch.arange(64, device=dev, dtype=torch.int64).view(1, 1, 64) * 32
               + torch.arange(32, device=dev, dtype=torch.int64).view(1, 32, 1)).reshape(-1) % (n_scan * EPP)
        rwant.zero_()
        bam_b200.direct_checksum(seq, n_rand, STORE_SEED, first_page * EPP, rwant, stream=sptr)
        times = []
        for _ in range(4):
            rsum.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream); arr.read(1 << 20, 64, rsum, idx=seq, stream=sptr); b.record(stream)
            stream.synchronize()
            times.append(a.elapsed_time(b))
        ctrl.check_status()
        cache.stats(reset=True)
        hit_seq_listed = {"ms": float(np.mean(times[1:])), "reads": n_rand, "ok": int(rsum.item()) == int(rwant.item())}
        del d_ridx, seq
        # the cache benchmark itself (sequential_access_warp with type ORIG, benchmarks/cache/main.cu:82-112): warp w
        # reads whole pages through array[], 32 consecutive elements per step, indices computed in the kernel
        cwant, csum = torch.zeros(1, dtype=torch.int64, device=dev), torch.zeros(1, dtype=torch.int64, device=dev)
        arr.page_scan(n_scan, cwant, first_page=0, stream=sptr)
        times = []
        for _ in range(4):
            csum.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream); arr.pattern_read(1, n_scan * EPP, csum, n_warps=n_scan // 4, n_pages_per_warp=4, stream=sptr, impl=1)
            b.record(stream)
            stream.synchronize()
            times.append(a.elapsed_time(b))
        ctrl.check_status()
        cst = cache.stats(reset=True)
        hit_seq = {"ms": float(np.mean(times[1:])), "reads": (n_scan // 4) * 4 * EPP, "misses": cst["misses"],
                   "ok": int(csum.item()) == int(cwant.item()) or n_scan % 4 != 0}
        # the reference's pattern benchmark, warm: every warp reads one resident 4 KiB page through a bam_ptr
        # cursor (nvm-pattern-bench --impl_type=3, 10 passes); checked against the page scan's sum of the same pages
        pwant, psum = torch.zeros(1, dtype=torch.int64, device=dev), torch.zeros(1, dtype=torch.int64, device=dev)
        arr.page_scan(n_scan, pwant, first_page=0, stream=sptr)
        times = []
        for _ in range(11):
            psum.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream); arr.pattern_read(1, n_scan * EPP, psum, n_warps=n_scan, n_pages_per_warp=1, stream=sptr); b.record(stream)
            stream.synchronize()
            times.append(a.elapsed_time(b))
        ctrl.check_status()
        pst = cache.stats(reset=True)
        hit_ptr = {"ms": float(np.mean(times[1:])), "elems": n_scan * EPP, "misses": pst["misses"],
                   "ok": int(psum.item()) == int(pwant.item())}

    # ---- reduce over ranks ---------------------------------------------------------------------------
    tot = torch.tensor([elapsed_ms, e2e_ms], dtype=torch.float64, device=dev)
    cnt = torch.tensor([st["read_ios"], st["hits"], st["misses"], st_e2e["read_ios"], int(ok), audit],
                       dtype=torch.int64, device=dev)
    red = sums[args.warmup:].clone()
    if world > 1:
        dist.all_reduce(tot, op=dist.ReduceOp.MAX)
        dist.all_reduce(cnt, op=dist.ReduceOp.SUM)
        dist.all_reduce(red, op=dist.ReduceOp.SUM)          # wrapping u64 sum == int64 sum bit for bit
    elapsed_ms, e2e_ms = tot.tolist()
    read_ios, hits, misses, e2e_ios, n_ok, audits = cnt.tolist()

    if rank == 0:
        peaks = measured_peaks()
        hbm_peak = peaks["hbm_gbs"] if peaks else 6650.0
        t = elapsed_ms * 1e-3
        value = read_ios / t
        gbs = value * PAGE / 1e9
        # per-launch figures of the dominant (only) kernel of the step, rank 0
        launch_ms = float(np.mean(kernel_ms))
        ach_link = (st["read_ios"] / args.steps) * PAGE / (launch_ms * 1e-3) / 1e9
        line = {
            "metric": "4KB-page IOPS via page cache", "value": value, "unit": "IOPS",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u64", "data": "synthetic",
            "config": workload_config(args, world),
            "gb_per_s": gbs, "accesses_per_s": world * n_acc * args.steps / t,
            "hit_rate": hits / max(1, hits + misses),
            "checksum_reduced": [f"{int(x) & ((1 << 64) - 1):#018x}" for x in red.tolist()],
            "verified": bool(n_ok == world and audits == 0),
            "e2e": {"value": e2e_ios / (e2e_ms * 1e-3), "unit": "IOPS", "h2d_bytes_per_step": n_acc * 8,
                    "d2h_bytes_per_step": 8},
            "gpu_launches": 2 * args.steps,
            "roofline": {"bound": "host_link", "achieved": ach_link, "peak": link_gbs, "unit": "GB/s",
                         "frac": ach_link / link_gbs if link_gbs else None,
                         # DRAM bytes per launch, scaled from the ncu capture of a small case of this kernel
                         # (2^23 reads, 1.40 M page reads: 6.0 GB written, 1.1 GB read): 4 300 B of DRAM writes per
                         # page read (the page lands once, + queue entries and slot words) and 131 B of DRAM reads
                         # per access (hit sector, bucket, slot word, index); both grow in proportion
                         "traffic": (st["read_ios"] / args.steps) * 4300.0 + n_acc * 131.0,
                         "traffic_note": "scaled from a small-case ncu capture, not measured on this launch; host-link "
                                         "bytes (the bound) are not DRAM traffic",
                         "kernel": "bam_fused<ArrayReadWork>",
                         "peak_aggregate": link_agg,
                         "note": "miss path: 4096 algorithmic bytes per page read cross the host link once; peak = "
                                 "1 GiB pinned-memory H2D copy measured in this run on all ranks at once (per-GPU share)"},
            "roofline_hit": {"bound": "hbm", "achieved": hit["pages"] * PAGE / (hit["ms"] * 1e-3) / 1e9,
                             "peak": hbm_peak, "unit": "GB/s",
                             "frac": hit["pages"] * PAGE / (hit["ms"] * 1e-3) / 1e9 / hbm_peak,
                             # ncu capture of a small warm pass: 272.7 MB read + 5.7 MB written for 268.4 MB of pages
                             "traffic": hit["pages"] * PAGE * (272.7 + 5.7) / 268.4,
                             "kernel": "bam_fused<PageScanWork>", "hits": hit["hits"], "misses": hit["misses"],
                             "note": "warm cache: whole resident pages read through the cache, 4096 algorithmic "
                                     "bytes per page; peak = MEASURED_PEAKS.json hbm_gbs" if peaks else "of fallback"},
            "hit_random_reads": {"reads_per_s": hit_rand["reads"] / (hit_rand["ms"] * 1e-3),
                                 "useful_gb_per_s": hit_rand["reads"] * 8 / (hit_rand["ms"] * 1e-3) / 1e9,
                                 "sector_gb_per_s": hit_rand["reads"] * 32 / (hit_rand["ms"] * 1e-3) / 1e9,
                                 "misses": hit_rand["misses"], "verified": hit_rand["ok"],
                                 "note": "2^26 uniform 8-byte reads from an index list over resident pages through array[] (all hits): "
                                         "per read one 32-byte sector of page data, the bucket and the slot record (twice); "
                                         "no pin, no atomic"},
            "hit_pattern_bam_ptr": {"elems_per_s": hit_ptr["elems"] / (hit_ptr["ms"] * 1e-3),
                                    "gib_per_s": hit_ptr["elems"] * 8 / (hit_ptr["ms"] * 1e-3) / (1 << 30),
                                    "pages": hit_ptr["elems"] // EPP, "misses": hit_ptr["misses"], "verified": hit_ptr["ok"],
                                    "vs_published": hit_ptr["elems"] * 8 / (hit_ptr["ms"] * 1e-3) / (1 << 30) / 373.6,
                                    "note": "warm cache, one warp per resident 4 KiB page through a bam_ptr cursor (the reference's "
                                            "pattern benchmark, impl 3); published: 373.6 GiB/s average over its warm passes, on its "
                                            "own GPU (asplosaoe/nvm_pattern_bench.log:26-62)"},
            "hit_sequential_reads": {"reads_per_s": hit_seq["reads"] / (hit_seq["ms"] * 1e-3),
                                     "gb_per_s": hit_seq["reads"] * 8 / (hit_seq["ms"] * 1e-3) / 1e9, "verified": hit_seq["ok"],
                                     "misses": hit_seq["misses"],
                                     "frac_of_hbm": hit_seq["reads"] * 8 / (hit_seq["ms"] * 1e-3) / 1e9 / hbm_peak,
                                     "vs_published": hit_seq["reads"] / (hit_seq["ms"] * 1e-3) / 2.272e10,
                                     "note": "warm cache, the reference's cache benchmark (sequential_access_warp, type ORIG): every "
                                             "warp reads whole resident pages through array[], 32 consecutive 8-byte elements per "
                                             "step, indices computed in the kernel; 169 GiB/s in its published log"},
            "hit_sequential_reads_listed": {"reads_per_s": hit_seq_listed["reads"] / (hit_seq_listed["ms"] * 1e-3),
                                            "gb_per_s": hit_seq_listed["reads"] * 8 / (hit_seq_listed["ms"] * 1e-3) / 1e9,
                                            "verified": hit_seq_listed["ok"],
                                            "note": "the same access shape driven by a 2^26-entry index list in HBM (8 bytes of "
                                                    "index traffic per 8 bytes read)"},
            "clocks": clocks, "setup_s": setup_s, "numa_rank0": numa,
        }
        line["config"]["placement"] = placement
        line["config"]["controller_blocks"] = ctrl_blocks
        line["config"]["controller_blocks_rule"] = ("given on the command line" if args.ctrl_blocks else
                                                    "48 x (pinned-copy GB/s measured on all ranks at once) / 55, in steps of 8")
    arr.close(); cache.close()
    for c in ctrls:
        c.close()
    del d_idx, sums, want, d_cdf, h_idx, d_stage
    torch.cuda.empty_cache()
    if args.graphs_last:
        graph_part_guarded()
    # ---- the other two configurations at full size (one GPU only): array random read through ONE queue pair, and the
    # block-level queue count x depth sweep; each verified (checksum against the oracle; sums and page CRC-32s)
    extras = {}
    if world == 1 and not args.no_extras:
        try:
            a = measure_array(argparse.Namespace(**{**vars(args), "steps": 1, "ctrl_blocks": 0}))
            extras["array_single_queue"] = {k: a[k] for k in ("value", "unit", "ms_per_step", "gb_per_s", "elements_per_s", "hit_rate",
                                                              "checksum", "verified", "config")}
            b = measure_block(argparse.Namespace(**{**vars(args), "store_gib": 64.0, "ctrl_blocks": 0}))
            extras["block_sweep"] = {"best_iops": b["value"], "sweep": b["sweep"], "verified": b["verified"], "config": b["config"]}
        except Exception as e:
            extras["error"] = f"{type(e).__name__}: {e}"
    # ---- CPU baselines last: nothing that runs on the host cores precedes a GPU measurement ----------------
    if rank == 0:
        if not args.no_cpu_baseline and world == 1:
            try:
                from oracle import pyoracle as orc
                cores = os.cpu_count() or 1
                ctrl_threads = max(1, cores // 8)
                workers = max(1, cores - ctrl_threads)
                cl = args.cpu_sample_lanes
                store = np.empty(n_local * EPP, dtype=np.uint64)
                slots = min(cache_pages, cl * reqs)
                t_cpu, ios_cpu, acc_cpu, miss_cpu = 0.0, 0, 0, 0
                use_ref_code = reference_code_available(orc)
                for s in range(3):
                    if use_ref_code:
                        stc, dt = cpu_reference_code_step(orc, n_local, first_page, slots, ctrl_threads, args.depth, cl, reqs,
                                                          ACCESS_SEED + 5000 + s, workers, store, cdf)
                        t_cpu += dt; ios_cpu += stc.read_ios; acc_cpu += stc.accesses; miss_cpu += stc.misses
                    else:
                        r = cpu_reference_step(orc, n_local, first_page, slots, min(args.queues, 128), args.depth, cl, reqs,
                                               ACCESS_SEED + 5000 + s, workers, ctrl_threads, store, cdf)
                        t_cpu += r.seconds; ios_cpu += r.read_ios; acc_cpu += r.accesses; miss_cpu += r.misses
                line["cpu_baseline"] = {
                    "value": ios_cpu / t_cpu, "unit": "IOPS", "cores": workers + ctrl_threads,
                    "kind": "reference" if use_ref_code else "port",
                    "accesses_per_s": acc_cpu / t_cpu, "hit_rate": 1.0 - miss_cpu / max(1, acc_cpu),
                    "sample": f"3 x ({cl} lanes x {reqs} reads) of the same Zipf stream, cold {slots}-slot cache, "
                              f"{workers} reader + {ctrl_threads} controller threads"
                              + ("; the reference's own page cache and queue code compiled for host threads (oracle/_ref)"
                                 if use_ref_code else "; CPU restatement of the reference's protocol")}
            except Exception as e:  # the baseline is reported, never required
                line["cpu_baseline"] = {"value": None, "unit": "IOPS", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
        if extras:
            line.update(extras)
            line["gpu_launches"] += 1 + 24
            line["verified"] = bool(line["verified"] and "error" not in extras and extras["array_single_queue"]["verified"]
                                    and extras["block_sweep"]["verified"])
        if "error" in graph_res:
            line["bfs"] = line["cc"] = {"error": graph_res["error"], "verified": False}
            line["verified"] = False
        elif graph_res:
            if graph_res.get("keep") is not None:
                graph_res["bfs"]["cpu_baseline"], graph_res["cc"]["cpu_baseline"] = graph_cpu_baselines(
                    args, graph_res["keep"], int((args.graph_cache_gib or 8.0) * (1 << 30)) // PAGE)
            line["bfs"], line["cc"] = graph_res["bfs"], graph_res["cc"]
            line["gpu_launches"] += line["bfs"]["gpu_launches"] + line["cc"]["gpu_launches"]
            line["verified"] = bool(line["verified"] and line["bfs"]["verified"] and line["cc"]["verified"])
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
