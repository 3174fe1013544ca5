#!/usr/bin/env python
"""Benchmark of the W4A4H MUL_MAT path:  python bench.py --gpus N --steps K --warmup W  [--impl reference]

Workload (config.workload): the 64-layer 27B-shaped decoder linear stack in W4A4H -- per layer q 5120->6144,
k 5120->1024, v 5120->1024, o 6144->5120, gate 5120->17408, up 5120->17408, down 17408->5120 -- run as M = 1 decode.
A step is one pass over all 448 matmuls; per layer four fp32 N(0,1) activations as in the decoder (q/k/v share one,
gate/up share one, o and down have their own) and matmuls that share an activation are one call; weights are synthetic
N(0, 0.02) rows rotated and quantized to W4A4H on the GPU (ruquant_b200.synth); 12.27 GB of weight blocks, so every
step streams far more than the 126 MB L2.  `value` is algorithmic GB/s: sum over matmuls of
N*(K/256)*144 + 4*M*K + 4*M*N bytes, divided by the step time, inputs resident in HBM.  `e2e` is the same pass
through the C ABI with host buffers: pinned-host -> device copies of the step's activations and device -> host
copies of its outputs inside the timed region.  `prefill` reports the M = 4096 gate/up-shaped GEMM
(K=5120, N=17408) in TOPS, whole node (rotate + quantize + tcgen05 GEMM + fold + epilogue).

With N GPUs the weight rows are sharded along N, the activations are replicated and each layer's output (its seven
matmul outputs side by side) is assembled on every rank: by default the kernels' epilogues store into every rank's
output buffer (mapped through symmetric memory) and one barrier kernel per layer closes the exchange; --gather nccl, or
a failed set-up, uses one NCCL all-gather per layer instead (total work fixed: "strong" scaling).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LAYER = [("q", 5120, 6144), ("k", 5120, 1024), ("v", 5120, 1024), ("o", 6144, 5120), ("gate", 5120, 17408),
         ("up", 5120, 17408), ("down", 17408, 5120)]
LAYER_DIMS = {name: (K, N) for name, K, N in LAYER}
GROUPS = [("q", "k", "v"), ("o",), ("gate", "up"), ("down",)]      # matmuls that share an activation
PREFILL = ("gate_up", 5120, 17408, 4096)
METRIC = "W4A4H decode GB/s @M=1 over the 64-layer 27B-shaped linear stack (prefill TOPS @M=4096 under 'prefill')"


def algorithmic_bytes(K, N, M):
    return N * (K // 256) * 144 + 4 * M * K + 4 * M * N


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 0.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        self.thread.join(timeout=2)
        sm = sorted(float(r[0]) for r in self.rows if len(r) >= 7 and r[0].replace(".", "").isdigit())
        mx = [float(r[1]) for r in self.rows if len(r) >= 7 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 7 and r[3 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------------- reference arm

def cpu_reference_layer(wb_host, x_host, threads):
    """One decoder layer's seven matmuls at M = 1 on the host cores with the reference's own compiled code
    (oracle/_ref) or, where that is absent, the oracle port.  Returns (seconds, kind)."""
    import oracle
    if oracle.have_ref():
        impl, kind = oracle.Ref(), "reference"
        run = lambda wb, K, x: impl.mul_mat(wb, 45, K, x, threads=threads)
    else:
        impl, kind = oracle.Port(), "port"
        run = lambda wb, K, x: impl.mul_mat(wb, 45, K, x, threads=threads)
    best = float("inf")
    for _ in range(3):
        t0 = time.perf_counter()
        for (name, K, N), wb, x in zip(LAYER, wb_host, x_host):
            run(wb, K, x)
        best = min(best, time.perf_counter() - t0)
    return best, kind


def host_layer(seed=0):
    """One layer of W4A4H weights quantized on the host by the oracle port (64 distinct rows per tensor, tiled, as
    the reference's own bench does to bound generation time) and its activations."""
    import numpy as np

    import oracle
    port = oracle.Port()
    rng = np.random.default_rng(seed)
    wbs, xs = [], []
    for name, K, N in LAYER:
        rows = port.quantize_weights(rng.normal(0, 0.02, (64, K)).astype(np.float32), 45)
        wbs.append(np.tile(rows, (N // 64, 1)))
        xs.append(rng.normal(0, 1, (1, K)).astype(np.float32))
    return wbs, xs


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    wbs, xs = host_layer()
    layer_bytes = sum(algorithmic_bytes(K, N, 1) for _, K, N in LAYER)
    times = []
    kind = None
    for i in range(args.warmup + args.steps):
        t, kind = cpu_reference_layer(wbs, xs, threads)
        if i >= args.warmup:
            times.append(t)
    t = sum(times) / len(times)
    gbs = layer_bytes / t / 1e9
    sample = "1 of 64 layers per step (7 matmuls, M=1), best of 3 per step; GB/s is per-layer bytes / per-layer time"
    line = {"impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int4 x int4 -> int32, fp32 epilogue", "data": "synthetic",
            "config": {"workload": "27B-shaped 64-layer W4A4H linear stack, M=1 decode (reference CPU path)", "layers_timed": 1},
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": kind, "sample": sample},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------- our arm

def run_ours(args):
    import torch
    import torch.distributed as dist

    import ruquant_b200 as rq
    from ruquant_b200 import synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rq.lib()
    hbm_peak, _, peak_kind = measured_peaks()
    L = args.layers

    # ---- the stack: rank r holds rows [r*N/g, (r+1)*N/g) of every tensor.  Per layer four activations, as in the
    # decoder: attention input -> q, k, v; attention output -> o; MLP input -> gate, up; MLP hidden -> down.  Weights
    # that share an activation go through one call (one rotate+quantize, one GEMV launch over all their row tiles),
    # the reference's fused launch for such matmuls (ggml_cuda_try_fuse).
    groups = []        # (K, x_dev, workspace, [(N_total, N_local, Weight, y_local, y_full)], gather or None)
    mats = []          # flat list of (K, N_total) for the byte count
    n_layer_local = sum(N // world for _n, _k, N in LAYER)
    # all activations of a pass in one device arena, all layer outputs in another: the end-to-end step is then one
    # pinned-host -> device copy and one device -> host copy around the captured graph
    k_layer = sum(LAYER_DIMS[names[0]][0] for names in GROUPS)
    x_arena = torch.empty((L * k_layer,), device=dev, dtype=torch.float32)
    # N > 1: every rank's output arena is mapped into every other rank (symmetric memory), and the decode GEMV's epilogue
    # writes its slice into all of them; one small barrier kernel per layer stands where the all-gather stood.  Falls
    # back to NCCL's all-gather when the mapping cannot be set up (or with --gather nccl).
    push = None
    if world > 1 and args.gather == "push":
        def all_agree(ok):      # a collective yes/no, so that the ranks never part ways
            flag = torch.tensor([1 if ok else 0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            return int(flag.item()) == 1

        why = ""
        try:
            import torch.distributed._symmetric_memory as symm
            y_arena = symm.empty(L * world * n_layer_local, dtype=torch.float32, device=dev)
            y_hdl = symm.rendezvous(y_arena, dist.group.WORLD)
            flags = symm.empty(64, dtype=torch.int32, device=dev)
            flags.zero_()
            f_hdl = symm.rendezvous(flags, dist.group.WORLD)
            order = [rank] + [r for r in range(world) if r != rank]          # own buffer first
            push = {"y_ptrs": [int(y_hdl.buffer_ptrs[r]) for r in order], "flag_ptrs": [int(p) for p in f_hdl.buffer_ptrs],
                    "epoch": torch.zeros(1, dtype=torch.int32, device=dev), "status": torch.zeros(1, dtype=torch.int32, device=dev),
                    "keep": (y_hdl, f_hdl, flags), "symm": symm, "order": order}
            torch.cuda.synchronize()
        except Exception as e:      # noqa: BLE001 -- any failure of the mapping means the NCCL path
            why, push = "%s: %s" % (type(e).__name__, e), None
        if not all_agree(push is not None):
            push = None
        if push is not None:
            # pre-flight on a tiny weight: every rank pushes 32 outputs into slot `rank` of every arena, meets the others
            # at the barrier kernel and must then hold what an NCCL all-gather of the same slices gives
            ran = True
            try:
                tw = rq.Weight(synth.random_weights(32, 256, rq.TYPE_W4A4, seed=5 + rank, device=dev).view(-1), rq.TYPE_W4A4, 256,
                               N=32, layouts=rq.PREPACK_DECODE)
                tx = torch.ones((1, 256), device=dev, dtype=torch.float32)
                rq.mul_mat_push([tw], tx, [[base + 4 * 32 * rank] for base in push["y_ptrs"]], [32], clip=1.0, act_group=64)
                rq.rank_barrier(push["flag_ptrs"], rank, push["epoch"], push["status"])
                torch.cuda.synchronize()
            except Exception as e:      # noqa: BLE001
                why, ran = "%s: %s" % (type(e).__name__, e), False
            if all_agree(ran):
                mine = y_arena[32 * rank:32 * rank + 32].clone()
                parts = [torch.empty_like(mine) for _ in range(world)]
                dist.all_gather(parts, mine)
                good = int(push["status"].item()) == 0 and bool(
                    (torch.cat(parts).view(torch.int32) == y_arena[:32 * world].view(torch.int32)).all().item())
                if not all_agree(good):
                    why, push = "pre-flight of the pushed outputs disagreed with the all-gather", None
            else:
                push = None
        if push is None and rank == 0:
            print("pushed outputs unavailable (%s); using the NCCL all-gather" % why, file=sys.stderr)
    if push is None:
        y_arena = torch.empty((L * world * n_layer_local,), device=dev, dtype=torch.float32)
    # the M = 4096 pass over the same stack needs the tensor-core operand of every weight as well (1 byte per weight)
    stack_layouts = rq.PREPACK_DECODE if (args.no_prefill or args.no_prefill_stack) else rq.PREPACK_ALL
    x_off = 0
    for layer in range(L):
        # the layer's seven local outputs sit side by side, so that one all-gather assembles the layer's output
        y_layer_all = y_arena[layer * world * n_layer_local:(layer + 1) * world * n_layer_local] if world > 1 else None
        if world == 1:
            y_layer_loc = y_arena[layer * n_layer_local:(layer + 1) * n_layer_local]
        elif push is not None:       # this rank's slot of the gathered layout, in place
            y_layer_loc = y_layer_all[rank * n_layer_local:(rank + 1) * n_layer_local]
        else:
            y_layer_loc = torch.empty((n_layer_local,), device=dev, dtype=torch.float32)
        col = 0
        for gi, names in enumerate(GROUPS):
            K = LAYER_DIMS[names[0]][0]
            g = torch.Generator(device=dev)
            g.manual_seed(7_000_000 + 10 * layer + gi)
            x = x_arena[x_off:x_off + K].view(1, K)
            x.copy_(torch.randn((1, K), generator=g, device=dev, dtype=torch.float32))
            x_off += K
            members = []
            for name in names:
                _, N = LAYER_DIMS[name]
                ti = [n for n, _k, _n in LAYER].index(name)
                nl = N // world
                blocks = synth.random_weights(nl, K, rq.TYPE_W4A4H, seed=100000 * layer + 100 * ti + rank, device=dev)
                w = rq.Weight(blocks.view(-1), rq.TYPE_W4A4H, K, N=nl, layouts=stack_layouts)
                w.blocks = None      # the kernels read only the prepacked stream
                del blocks
                y_loc = y_layer_loc[col:col + nl].view(1, nl)
                col += nl
                members.append((N, nl, w, y_loc, y_loc))
                mats.append((K, N))
            last = gi == len(GROUPS) - 1
            dst = None
            if push is not None:      # element offset of each member's output inside every rank's arena
                offs, c0 = [], col - sum(m[1] for m in members)
                for m in members:
                    offs.append((layer * world + rank) * n_layer_local + c0)
                    c0 += m[1]
                dst = [[base + 4 * o for o in offs] for base in push["y_ptrs"]]
            groups.append((K, x, rq.new_workspace(K, 1, dev), members,
                           (y_layer_all, y_layer_loc) if (world > 1 and last) else None, dst))
    torch.cuda.synchronize()
    # algorithmic bytes: every weight block and every output once, every activation once per group that shares it
    total_bytes = sum(N * (K // 256) * 144 + 4 * N for (K, N) in mats) + sum(4 * g[0] for g in groups)
    stream = torch.cuda.Stream(device=dev)

    def enqueue_pass(quantize=True, layers=None):
        per_layer = len(GROUPS)
        sel = groups if layers is None else groups[layers[0] * per_layer:layers[1] * per_layer]
        for K, x, ws, members, gather, dst in sel:
            weights = [m[2] for m in members]
            outs = [m[3] for m in members]
            if not quantize:           # the GEMV launches alone, on this rank's shards: no exchange
                rq.mul_mat_quantized(weights, 1, ws, out=outs, act_group=64, stream=stream)
                continue
            if dst is not None:
                rq.mul_mat_push(weights, x, dst, [m[1] for m in members], clip=1.0, act_group=64, workspace=ws, stream=stream)
            else:
                rq.mul_mat(weights, x, out=outs, clip=1.0, act_group=64, workspace=ws, stream=stream)
            if gather is not None:       # end of a layer: every rank gets every rank's slice of the layer's output
                if push is not None:
                    rq.rank_barrier(push["flag_ptrs"], rank, push["epoch"], push["status"], stream=stream)
                else:
                    dist.all_gather_into_tensor(gather[0], gather[1])

    def capture(fn):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            fn()                      # warm: first-launch attribute set-up happens outside capture
            stream.synchronize()
            with torch.cuda.graph(g, stream=stream):
                fn()
        return g

    g_pass = capture(lambda: enqueue_pass(True))
    if push is not None:
        # one pass has run (the capture's warm-up): the pushed arena must equal what NCCL's all-gather assembles from the
        # ranks' own slots, bit for bit, and no barrier may have run out of time
        torch.cuda.synchronize()
        dist.barrier()
        ya = y_arena.view(L, world, n_layer_local)
        mine = ya[:, rank].contiguous()
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        ref_arena = torch.stack(parts, dim=1)
        same = bool((ref_arena.view(torch.int32) == ya.view(torch.int32)).all().item()) and int(push["status"].item()) == 0
        flag = torch.tensor([1 if same else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) != 1:
            push["check"] = "FAILED: pushed outputs differ from the all-gathered ones (or a barrier timed out)"
            if rank == 0:
                print(push["check"], file=sys.stderr)
    g_gemv = capture(lambda: enqueue_pass(False))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                fn()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                fn()
            e1.record(stream)
            barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    sampler = ClockSampler(local) if rank == 0 else None
    ms_step = timed(g_pass.replay, args.steps, args.warmup)
    clocks = sampler.stop() if sampler else None
    value = total_bytes / (ms_step * 1e-3) / 1e9

    # ---- dominant kernel alone: the 448 GEMV launches on already-quantized activations
    roofline = None
    if g_gemv is not None:
        ms_gemv = timed(g_gemv.replay, args.steps, args.warmup)
        achieved = total_bytes / world / (ms_gemv * 1e-3) / 1e9        # per GPU: each rank streams 1/world of the weights
        # DRAM traffic per launch: an ncu capture of the K=5120 N=17408 launch read 44.65 MB for a 44.56 MB decode stream,
        # i.e. the stream once; scaled to the stack's average launch by stream bytes
        stream_bytes = sum(((N // world + 15) // 16) * 16 * K // 2 for (K, N) in mats)
        traffic = 1.002 * stream_bytes / len(groups)
        roofline = {"bound": "hbm", "kernel": "rq_gemv_mma_kernel", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                    "frac": achieved / hbm_peak, "peak_kind": "of " + peak_kind, "frac_of_nominal_8000": achieved / 8000.0,
                    "avg_launch_us": ms_gemv * 1e3 / len(groups), "launches_per_step": len(groups),
                    "algorithmic_bytes_per_launch": total_bytes / world / len(groups), "traffic": traffic, "per_gpu": True,
                    "traffic_note": "dram read+write bytes per launch, ncu capture of one shape scaled by stream bytes"}

    # ---- end to end through the C ABI with host buffers
    x_host = torch.randn((L * k_layer,), dtype=torch.float32).pin_memory()
    # every rank needs all the activations; of the outputs each rank takes only its own rows' share to the host (the
    # gathered copy on the device is what the next node would read)
    y_host = torch.empty((L, n_layer_local) if world > 1 else (L * n_layer_local,), dtype=torch.float32).pin_memory()
    h2d = x_host.numel() * 4
    d2h = y_host.numel() * 4

    # The pass is cut into chunks of layers, each its own graph: the input copy of chunk i+1 and the output copy of
    # chunk i-1 run on two copy streams beside chunk i.  Every step starts after the previous one has ended (copies
    # included) and ends with its last output copy, so nothing of a step lies outside its timed region.
    n_chunks = min(8, L)
    bounds = [round(i * L / n_chunks) for i in range(n_chunks + 1)]
    g_chunks = [capture(lambda a=bounds[i], b=bounds[i + 1]: enqueue_pass(True, (a, b))) for i in range(n_chunks)]
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    ev_in = [torch.cuda.Event() for _ in range(n_chunks)]
    ev_done = [torch.cuda.Event() for _ in range(n_chunks)]
    y_layer = world * n_layer_local

    def e2e_step():
        s_in.wait_stream(stream)
        s_out.wait_stream(stream)
        for i in range(n_chunks):
            a, b = bounds[i], bounds[i + 1]
            with torch.cuda.stream(s_in):
                x_arena[a * k_layer:b * k_layer].copy_(x_host[a * k_layer:b * k_layer], non_blocking=True)
                ev_in[i].record(s_in)
            stream.wait_event(ev_in[i])
            g_chunks[i].replay()
            ev_done[i].record(stream)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[i])
                if world > 1:
                    y_host[a:b].copy_(y_arena.view(L, world, n_layer_local)[a:b, rank], non_blocking=True)
                else:
                    y_host[a * y_layer:b * y_layer].copy_(y_arena[a * y_layer:b * y_layer], non_blocking=True)
        stream.wait_stream(s_out)

    ms_e2e = timed(e2e_step, args.steps, args.warmup)
    e2e = {"value": total_bytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "ms_per_step": ms_e2e, "copy_overlap": "%d layer chunks, copies on two streams beside the compute" % n_chunks,
           "per_rank": "every rank copies all activations in and its own share of the outputs out" if world > 1 else None}

    # ---- prefill: the M = 4096 gate/up-shaped and down-shaped GEMMs, whole node and GEMM kernel alone
    prefill = None
    if not args.no_prefill:
        def prefill_leg(K, N, M, seed, with_cpu):
            nl = N // world
            blocks = synth.random_weights(nl, K, rq.TYPE_W4A4H, seed=seed + rank, device=dev)
            w = rq.Weight(blocks.view(-1), rq.TYPE_W4A4H, K, N=nl, layouts=rq.PREPACK_PREFILL)
            g = torch.Generator(device=dev)
            g.manual_seed(99)
            x = torch.randn((M, K), generator=g, device=dev, dtype=torch.float32)
            y = torch.empty((M, nl), device=dev, dtype=torch.float32)
            ws = rq.new_workspace(K, M, dev)
            y_all, dst = None, None
            if world > 1 and push is not None:
                # the gathered [M][N] output of every rank, mapped everywhere: the GEMM's final store writes this rank's
                # columns into all of them while the MMAs of the next unit run; then one barrier kernel
                y_all = push["symm"].empty(M * N, dtype=torch.float32, device=dev)
                hdl = push["symm"].rendezvous(y_all, dist.group.WORLD)
                dst = [[int(hdl.buffer_ptrs[r]) + 4 * rank * nl] for r in push["order"]]
            elif world > 1:
                y_all = torch.empty((world, M, nl), device=dev, dtype=torch.float32)

            # N > 1: the ranks share the rotate+quantize work too -- rank r does tokens [r*M/g, (r+1)*M/g), the ranks exchange
            # the one-byte codes, group multipliers and token units (M*K bytes and a little, a quarter of what x itself
            # would take; identical bits by construction), then every rank multiplies all tokens by its own rows
            # (worth it where the rotation is expensive: at K = 17408, 315 us replicated, the node takes 0.566 ms shared against
            # 0.707 replicated on 4 GPUs; at K = 5120, 74 us replicated, 0.493 against 0.497)
            share = (world > 1 and dst is not None and M % world == 0 and not args.replicated_quantizer and
                     K * max(w.desc.had_p, 1) >= args.share_threshold)
            if share:
                # the workspace lives in memory mapped into every rank: one copy kernel carries this rank's rows to the others
                from ruquant_b200 import shard
                ws = rq.init_workspace(push["symm"].empty(rq.workspace_bytes(K, M), dtype=torch.uint8, device=dev), K, M)
                ws_hdl = push["symm"].rendezvous(ws, dist.group.WORLD)
                ws_ptrs = [int(p) for p in ws_hdl.buffer_ptrs]
                t0, t1 = shard.token_range(M, rank, world)
                fmt = rq.act_format(w, M)
                torch.cuda.synchronize()
                dist.barrier()

            def node():
                if share:
                    rq.quantize_rows(x[t0:t1], M, t0, w.n_rot, 1.0, 64, fmt, ws, stream=stream)
                    rq.share_rows(ws_ptrs, rank, ws.numel(), K, M, 64, t0, t1 - t0, stream=stream)
                    rq.rank_barrier(push["flag_ptrs"], rank, push["epoch"], push["status"], stream=stream)
                    rq.mul_mat_push([w], None, dst, [N], act_group=64, workspace=ws, stream=stream, M=M)
                    # (this barrier also stands between the ranks' reads of the workspaces and the next step's rows)
                    rq.rank_barrier(push["flag_ptrs"], rank, push["epoch"], push["status"], stream=stream)
                    return
                if dst is not None:
                    rq.mul_mat_push([w], x, dst, [N], clip=1.0, act_group=64, workspace=ws, stream=stream)
                    rq.rank_barrier(push["flag_ptrs"], rank, push["epoch"], push["status"], stream=stream)
                    return
                rq.mul_mat(w, x, out=y, clip=1.0, act_group=64, workspace=ws, stream=stream)
                if world > 1:
                    dist.all_gather_into_tensor(y_all.view(-1), y.view(-1))

            def local_node():        # this rank's share without the exchange: the compute-only curve
                rq.mul_mat(w, x, out=y, clip=1.0, act_group=64, workspace=ws, stream=stream)

            def gemm_only():
                rq.mul_mat_quantized(w, M, ws, out=y, act_group=64, stream=stream)

            def nofold():
                rq.tc_nofold_probe(w, M, ws, y, stream=stream)

            reps = max(3, args.steps)
            ms_node = timed(node, reps, 3)
            if dst is not None:
                # the pushed [M][N] must hold, in this rank's columns, what the plain node computes, on every rank
                torch.cuda.synchronize()
                dist.barrier()
                with torch.cuda.stream(stream):
                    rq.mul_mat(w, x, out=y, clip=1.0, act_group=64, workspace=ws, stream=stream)
                stream.synchronize()
                parts = [torch.empty_like(y) for _ in range(world)]
                dist.all_gather(parts, y)
                same = bool((torch.cat(parts, dim=1).view(torch.int32) == y_all.view(M, N).view(torch.int32)).all().item())
                same = same and int(push["status"].item()) == 0
                flag = torch.tensor([1 if same else 0], device=dev)
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                if int(flag.item()) != 1:
                    push["check"] = "FAILED: prefill pushed output differs from the all-gathered one"
                    if rank == 0:
                        print(push["check"], file=sys.stderr)
            ms_local = timed(local_node, reps, 3) if world > 1 else ms_node
            ms_gemm = timed(gemm_only, reps, 3)
            ms_probe = timed(nofold, reps, 3)
            with torch.cuda.stream(stream):
                local_node()             # leave a real result in y for the checks below
            stream.synchronize()
            rq.device_status(ws, K, M)
            ops = 2.0 * M * N * K
            tops_gemm = 2.0 * M * nl * K / (ms_gemm * 1e-3) / 1e12 * world
            tops_probe = 2.0 * M * nl * K / (ms_probe * 1e-3) / 1e12 * world
            out = {"workload": "W4A4H K=%d N=%d M=%d" % (K, N, M), "tops_node": ops / (ms_node * 1e-3) / 1e12, "ms_node": ms_node,
                   "ms_node_compute_only": ms_local, "tops_node_compute_only": ops / (ms_local * 1e-3) / 1e12,
                   "nvlink_bytes_out_per_rank": (world - 1) * M * nl * 4,
                   "quantizer": "shared: each rank quantizes M/%d tokens, codes exchanged (%d bytes in per rank)" % (
                       world, (world - 1) * (M // world) * (K + 4 * (K // 64) + 4)) if share else "replicated on every rank",
                   "tops_gemm_kernel": tops_gemm, "ms_gemm_kernel": ms_gemm,
                   "int8_dense_peak_nominal_tops": 4500.0 * world,
                   "frac_of_nominal_int8_peak": ops / (ms_node * 1e-3) / 1e12 / (4500.0 * world),
                   # the dominant kernel against the tensor-core bound: nominal dense 8-bit peak, and what this kernel's own
                   # TMA / tcgen05 / TMEM pipeline reaches in the same run with the per-group fold left out (one
                   # accumulator over all of K: rq_w4a4_tc_nofold_probe)
                   "roofline": {"bound": "tensor", "kernel": "rq_gemm_tc_kernel", "achieved": tops_gemm, "peak": 4500.0 * world,
                                "unit": "TOP/s", "frac": tops_gemm / (4500.0 * world), "peak_kind": "nominal dense int8/fp8 (no measured 8-bit peak in MEASURED_PEAKS.json)",
                                "peak_measured_nofold": tops_probe, "frac_of_measured_nofold": tops_gemm / tops_probe,
                                "algorithmic_ops_per_launch": 2.0 * M * nl * K, "fold_fmas_per_launch": M * nl * K / 64.0,
                                "avg_launch_us": ms_gemm * 1e3, "traffic": None}}
            if with_cpu and world == 1:
                # end to end through the C ABI with host buffers: x from pinned host memory, y back to it, every step
                xh = x.cpu().pin_memory()
                yh = torch.empty((M, nl), dtype=torch.float32).pin_memory()

                def e2e_node():
                    x.copy_(xh, non_blocking=True)
                    rq.mul_mat(w, x, out=y, clip=1.0, act_group=64, workspace=ws, stream=stream)
                    yh.copy_(y, non_blocking=True)

                ms_e2e_p = timed(e2e_node, reps, 3)
                out["e2e"] = {"value": ops / (ms_e2e_p * 1e-3) / 1e12, "unit": "TOP/s", "ms_per_step": ms_e2e_p,
                              "h2d_bytes_per_step": M * K * 4, "d2h_bytes_per_step": M * nl * 4}
                if not args.no_cpu:
                    # the reference's CPU node on the first 64 tokens (its scalar dot product makes 4096 tokens a matter of
                    # minutes); every output of those tokens is also compared with what the GPU left in y
                    import oracle
                    tok = 64
                    wb_host = blocks.cpu().numpy()
                    x_host = xh[:tok].numpy()
                    impl, kind = (oracle.Ref(), "reference") if oracle.have_ref() else (oracle.Port(), "port")
                    threads = os.cpu_count() or 1
                    best, y_cpu = float("inf"), None
                    for _ in range(2):
                        t0 = time.perf_counter()
                        y_cpu = impl.mul_mat(wb_host, 45, K, x_host, threads=threads)
                        best = min(best, time.perf_counter() - t0)
                    same = bool((y_cpu.view("uint32") == yh[:tok].numpy().view("uint32")).all())
                    out["cpu_baseline"] = {"value": 2.0 * tok * N * K / best / 1e12, "unit": "TOP/s", "cores": threads, "kind": kind,
                                           "sample": "first %d of %d tokens, best of 2; %.3f s measured, %.1f s for all tokens by linear "
                                                     "extrapolation" % (tok, M, best, best * M / tok),
                                           "bit_identical_to_gpu_on_sample": same}
            del blocks
            return out

        _, K, N, M = PREFILL
        prefill = prefill_leg(K, N, M, 424242, True)
        prefill["down_shaped"] = prefill_leg(N, K, M, 434343, False)      # K = 17408 (68 x 256 rotation), N = 5120

    # ---- configuration 5 at M = 4096: one pass over the whole stack (1.787e14 operations at 64 layers).  The linears are
    # not chained: every activation width has one seeded N(0,1) input, every output width one buffer.  N-sharded ranks
    # assemble every matmul's output on every rank: the GEMM's copy warps store each finished unit into the other ranks'
    # gathered [M][N] buffers while the next units fold, one barrier kernel per layer (an NCCL all-gather after every
    # matmul where the buffers cannot be mapped).
    prefill_stack = None
    if not args.no_prefill and not args.no_prefill_stack:
        Mp = PREFILL[3]
        xs, wss, ys, yg = {}, {}, {}, {}
        for names in GROUPS:
            K = LAYER_DIMS[names[0]][0]
            if K not in xs:
                g = torch.Generator(device=dev)
                g.manual_seed(4096 + K)
                xs[K] = torch.randn((Mp, K), generator=g, device=dev, dtype=torch.float32)
                wss[K] = rq.new_workspace(K, Mp, dev)
            for name in names:
                N = LAYER_DIMS[name][1]
                if N not in ys:
                    ys[N] = torch.empty((Mp, N // world), device=dev, dtype=torch.float32)
                    if world > 1:
                        yg[N] = torch.empty((world, Mp, N // world), device=dev, dtype=torch.float32)

        ygs, ygp = {}, {}       # gathered [M][N] outputs mapped into every rank, and their addresses (own buffer first)
        if push is not None:
            for name, _k, N in LAYER:      # one gathered buffer per tensor of the layer
                ygs[name] = push["symm"].empty(Mp * N, dtype=torch.float32, device=dev)
                hdl = push["symm"].rendezvous(ygs[name], dist.group.WORLD)
                ygp[name] = [int(hdl.buffer_ptrs[r]) for r in push["order"]]
            torch.cuda.synchronize()
            dist.barrier()

        def stack_pass(gather):
            for i, (K, _x, _ws, members, _g, _dst) in enumerate(groups):
                weights = [m[2] for m in members]
                if gather and push is not None:
                    names = GROUPS[i % len(GROUPS)]
                    rq.mul_mat_push(weights, xs[K], [[ygp[nm][d] + 4 * rank * m[1] for nm, m in zip(names, members)] for d in range(world)],
                                    [m[0] for m in members], clip=1.0, act_group=64, workspace=wss[K], stream=stream)
                    if i % len(GROUPS) == len(GROUPS) - 1:
                        rq.rank_barrier(push["flag_ptrs"], rank, push["epoch"], push["status"], stream=stream)
                    continue
                outs = [ys[m[0]] for m in members]
                rq.mul_mat(weights, xs[K], out=outs, clip=1.0, act_group=64, path=rq.PATH_TC, workspace=wss[K], stream=stream)
                if gather and world > 1:
                    for m in members:
                        dist.all_gather_into_tensor(yg[m[0]].view(-1), ys[m[0]].view(-1))

        ops_stack = sum(2.0 * Mp * N * K for (K, N) in mats)
        ms_stack = timed(lambda: stack_pass(True), 2, 1)
        ms_stack_local = timed(lambda: stack_pass(False), 2, 1) if world > 1 else ms_stack
        for K in wss:
            rq.device_status(wss[K], K, Mp)
        stack_check = None
        if push is not None:
            # what the last down projection left in every rank's gathered buffer against an NCCL all-gather of the slices
            Nd = LAYER_DIMS["down"][1]
            nl = Nd // world
            mine = ygs["down"].view(Mp, Nd)[:, rank * nl:(rank + 1) * nl].contiguous()
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine)
            same = bool((torch.cat(parts, dim=1).view(torch.int32) == ygs["down"].view(Mp, Nd).view(torch.int32)).all().item())
            flag = torch.tensor([1 if same and int(push["status"].item()) == 0 else 0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            stack_check = "equal" if int(flag.item()) == 1 else "FAILED"
        prefill_stack = {"workload": "%d-layer stack, M=%d prefill, 7 matmuls per layer (%.4g operations per pass)" % (L, Mp, ops_stack),
                         "ms_per_pass": ms_stack, "tops": ops_stack / (ms_stack * 1e-3) / 1e12,
                         "ms_per_pass_compute_only": ms_stack_local, "tops_compute_only": ops_stack / (ms_stack_local * 1e-3) / 1e12,
                         "frac_of_nominal_int8_peak": ops_stack / (ms_stack * 1e-3) / 1e12 / (4500.0 * world),
                         "nvlink_bytes_in_per_rank_per_pass": (world - 1) * sum(Mp * (N // world) * 4 for (_k, N) in mats),
                         "exchange": "none" if world == 1 else ("outputs stored into every rank's gathered buffers by the GEMM's copy "
                                                                "warps, one barrier kernel per layer" if push is not None else
                                                                "ncclAllGather per matmul output"),
                         "pushed_vs_all_gather": stack_check}
        # ---- the same pass in the reference's own tensor-parallel arrangement (src/convert.rs:120-128, mxpatch:5293-5374):
        # q/k/v and gate/up stay split along N and nothing is gathered (their consumers are sharded the same way), o and
        # down are split along K (block-diagonal rotation): every rank multiplies its slice of x by its block columns and
        # the partial outputs are added in rank order over peer-mapped buffers.  A K slice that is not a whole number of
        # blocks with a factorable length (down on 8 ranks: 2176 inputs) stays split along N with its all-gather.
        if world > 1 and push is not None:
            symm = push["symm"]
            two_shot = world > 2
            ksplit = {}
            for name in ("o", "down"):
                K, N = LAYER_DIMS[name]
                ks = K // world
                if K % world or ks % 256 or rq.hadamard_factor(ks) is None:
                    continue
                g = torch.Generator(device=dev)
                g.manual_seed(9000 + rank + 16 * len(ksplit))
                part = symm.empty(Mp * N, dtype=torch.float32, device=dev)
                yk = symm.empty(Mp * N, dtype=torch.float32, device=dev)
                ksplit[name] = {"ks": ks, "N": N, "x": torch.randn((Mp, ks), generator=g, device=dev, dtype=torch.float32),
                                "ws": rq.new_workspace(ks, Mp, dev), "part": part, "y": yk,
                                "pptrs": [int(p) for p in symm.rendezvous(part, dist.group.WORLD).buffer_ptrs],
                                "yptrs": [int(p) for p in symm.rendezvous(yk, dist.group.WORLD).buffer_ptrs], "w": []}
                for layer in range(L):
                    blocks = synth.random_weights(N, ks, rq.TYPE_W4A4H, seed=8_000_000 + 100 * layer + rank, device=dev)
                    wk_ = rq.Weight(blocks.view(-1), rq.TYPE_W4A4H, ks, N=N, layouts=rq.PREPACK_PREFILL)
                    wk_.blocks = None
                    del blocks
                    ksplit[name]["w"].append(wk_)

            def ranks_meet():
                rq.rank_barrier(push["flag_ptrs"], rank, push["epoch"], push["status"], stream=stream)

            def tp_pass(exchange):
                for i, (K, _x, _ws, members, _g, _dst) in enumerate(groups):
                    name = GROUPS[i % len(GROUPS)][0]
                    ksp = ksplit.get(name) if len(members) == 1 else None
                    if ksp is None:
                        rq.mul_mat([m[2] for m in members], xs[K], out=[ys[m[0]] for m in members], clip=1.0, act_group=64,
                                   path=rq.PATH_TC, workspace=wss[K], stream=stream)
                        if exchange and len(members) == 1:       # o / down that could not be split along K
                            dist.all_gather_into_tensor(yg[members[0][0]].view(-1), ys[members[0][0]].view(-1))
                        continue
                    N = ksp["N"]
                    rq.mul_mat(ksp["w"][i // len(GROUPS)], ksp["x"], out=ksp["part"].view(Mp, N), clip=1.0, act_group=64,
                               path=rq.PATH_TC, workspace=ksp["ws"], stream=stream)
                    if not exchange:
                        continue
                    # o and down have partial buffers of their own and alternate: the barrier ahead of one's sum is also
                    # the barrier after the other's, so a one-shot sum needs no second one while both are split along K
                    ranks_meet()
                    rq.sum_partials(ksp["pptrs"], rank, Mp * N, ksp["yptrs"] if two_shot else
                                    [p if r == rank else 0 for r, p in enumerate(ksp["yptrs"])], two_shot=two_shot, stream=stream)
                    if two_shot or len(ksplit) < 2:
                        ranks_meet()

            ms_tp = timed(lambda: tp_pass(True), 2, 1)
            ms_tp_local = timed(lambda: tp_pass(False), 2, 1)
            chk = []
            for name, ksp in ksplit.items():
                rq.device_status(ksp["ws"], ksp["ks"], Mp)
                got = [torch.empty_like(ksp["y"]) for _ in range(world)]
                dist.all_gather(got, ksp["y"])
                chk.append(all(bool((c.view(torch.int32) == ksp["y"].view(torch.int32)).all().item()) for c in got))
            n_sum = (2.0 * (world - 1) / world if two_shot else float(world - 1))
            prefill_stack["tensor_parallel"] = {
                "arrangement": "q/k/v, gate/up split along N, outputs left sharded; %s split along K, partial outputs added in rank "
                               "order (%s)" % (", ".join(sorted(ksplit)) or "no tensor", "two-shot" if two_shot else "one-shot"),
                "n_split_with_all_gather": [n for n in ("o", "down") if n not in ksplit],
                "ms_per_pass": ms_tp, "tops": ops_stack / (ms_tp * 1e-3) / 1e12,
                "ms_per_pass_compute_only": ms_tp_local, "tops_compute_only": ops_stack / (ms_tp_local * 1e-3) / 1e12,
                "frac_of_nominal_int8_peak": ops_stack / (ms_tp * 1e-3) / 1e12 / (4500.0 * world),
                "nvlink_bytes_in_per_rank_per_pass": int(L * sum(n_sum * Mp * k["N"] * 4 for k in ksplit.values())),
                "all_ranks_bit_identical": all(chk) and int(push["status"].item()) == 0,
                "note": "a K-split rank quantizes its slice of x with its own range, in the reference as here: the sums are not "
                        "the one-GPU outputs (the N split's are)"}
            del ksplit
        del xs, wss, ys, yg, ygs

    # ---- the reference's own tensor-parallel mode for attn_output / ffn_down: weights split along K (block-diagonal
    # rotation, `--rot-blocks`), every rank multiplies its slice of x by its block columns, the partial outputs are added in
    # rank order over peer-mapped buffers (rq_w4a4_sum_partials) -- beside the N-split of the same shapes above
    k_split = None
    if world > 1 and push is not None and not args.no_prefill:
        k_split = []
        symm = push["symm"]
        for name in ("o", "down"):
            K, N = LAYER_DIMS[name]
            ks = K // world
            if ks % 256 or rq.hadamard_factor(ks) is None:
                continue
            blocks = synth.random_weights(N, ks, rq.TYPE_W4A4H, seed=515151 + rank, device=dev)     # a slice is a W4A4H tensor of its own
            wk_ = rq.Weight(blocks.view(-1), rq.TYPE_W4A4H, ks, N=N, layouts=rq.PREPACK_ALL)
            del blocks
            for Mk in (1, PREFILL[3]):
                g = torch.Generator(device=dev)
                g.manual_seed(777 + rank)
                xk = torch.randn((Mk, ks), generator=g, device=dev, dtype=torch.float32)
                part = symm.empty(Mk * N, dtype=torch.float32, device=dev)
                ph = symm.rendezvous(part, dist.group.WORLD)
                yk = torch.empty((Mk, N), device=dev, dtype=torch.float32)
                wsk = rq.new_workspace(ks, Mk, dev)
                pptrs = [int(p) for p in ph.buffer_ptrs]
                yptrs = [yk.data_ptr() if r == rank else 0 for r in range(world)]

                def knode():
                    rq.mul_mat(wk_, xk, out=part.view(Mk, N), clip=1.0, act_group=64, workspace=wsk, stream=stream)
                    rq.rank_barrier(push["flag_ptrs"], rank, push["epoch"], push["status"], stream=stream)
                    rq.sum_partials(pptrs, rank, Mk * N, yptrs, stream=stream)
                    rq.rank_barrier(push["flag_ptrs"], rank, push["epoch"], push["status"], stream=stream)    # partials free again

                def klocal():
                    rq.mul_mat(wk_, xk, out=part.view(Mk, N), clip=1.0, act_group=64, workspace=wsk, stream=stream)

                reps = max(3, args.steps)
                ms_k = timed(knode, reps, 3)
                ms_kl = timed(klocal, reps, 3)
                # all ranks must hold the same bits
                chk = [torch.empty_like(yk) for _ in range(world)]
                dist.all_gather(chk, yk)
                same = all(bool((c.view(torch.int32) == yk.view(torch.int32)).all().item()) for c in chk) and int(push["status"].item()) == 0
                k_split.append({"tensor": name, "K": K, "N": N, "M": Mk, "ms_node": ms_k, "ms_node_compute_only": ms_kl,
                                "nvlink_bytes_in_per_rank": (world - 1) * Mk * N * 4, "all_ranks_bit_identical": same,
                                "n_split_nvlink_bytes_out_per_rank": (world - 1) * Mk * (N // world) * 4})
            del wk_

    # ---- the reference's own performance shapes (one GPU): decode widths in GB/s, 512 tokens in TOPS
    perf_shapes = None
    if rank == 0 and world == 1 and not args.no_perf_shapes:
        perf_shapes = []
        for rows, tokens, K in REF_PERF_SHAPES:
            r = time_shape(K, rows, tokens, rq.TYPE_W4A4H, 0, 64, 5, 2, probe=False)
            perf_shapes.append({"rows": rows, "tokens": tokens, "K": K, "us_node": r["us_node"], "us_contraction": r["us_contraction"],
                                "GBps_node": r["GBps_node"], "frac_hbm_node": r["frac_hbm_node"], "TOPS_node": r["TOPS_node"]})

    # ---- CPU baseline beside it (rank 0, one GPU): one layer on the host cores
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        wbs, xs = host_layer()
        threads = os.cpu_count() or 1
        t, kind = cpu_reference_layer(wbs, xs, threads)
        layer_bytes = sum(algorithmic_bytes(K, N, 1) for _, K, N in LAYER)
        cpu = {"value": layer_bytes / t / 1e9, "unit": "GB/s", "cores": threads, "kind": kind,
               "sample": "1 of 64 layers (7 matmuls, M=1), best of 3; per-layer bytes / per-layer time"}

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "int4 x int4 -> int32, fp32 epilogue", "data": "synthetic",
                "config": {"workload": "27B-shaped %d-layer W4A4H linear stack, M=1 decode, 7 matmuls per layer" % L,
                           "weights_gb": sum(N * (K // 256) * 144 for (K, N) in mats) / 1e9,
                           "activation_sharing": "q,k,v | o | gate,up | down: one rotate+quantize and one GEMV launch per group",
                           "l2": "inputs larger than L2 (weights streamed once per step)",
                           "parallelism": ("single GPU" if world == 1 else
                                           "N-sharded x%d, GEMV epilogues store into every rank's output over NVLink, one barrier kernel "
                                           "per layer (check against an NCCL all-gather: %s)" % (world, push.get("check", "equal")) if push is not None else
                                           "N-sharded x%d, one NCCL all-gather per layer output" % world),
                           "cuda_graph": True,
                           "reference_arm": "bench.py --impl reference times 1 of the 64 layers per step on the host cores (GB/s is "
                                            "per-layer bytes / per-layer time, so the two arms' values compare; their ms_per_step do not)"},
                "frac_of_hbm_peak": value / (hbm_peak * world), "peak_kind": "of " + peak_kind,
                "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "prefill": prefill, "prefill_stack": prefill_stack,
                "reference_perf_shapes": perf_shapes, "k_split": k_split, "clocks": clocks,
                # kernels of this library launched inside the timed decode region: a rotate+quantize and a GEMV per
                # activation group, and one barrier kernel per layer when the ranks push their outputs
                "gpu_launches": (2 * len(groups) + (L if push is not None else 0)) * args.steps}
        print(json.dumps(line))
    if world > 1:
        # every rank is past its last collective: leave without tearing NCCL down under the captured graphs
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def run_wquant(args):
    """The GPU weight quantizer on N rows of K against the reference's CPU quantizer on a sample of the same rows."""
    import torch

    import oracle
    import ruquant_b200 as rq

    parts = [int(v) for v in args.wquant.split(",")]
    K, N = parts[:2]
    type_ = parts[2] if len(parts) > 2 else rq.TYPE_W4A4H
    wgroup = parts[3] if len(parts) > 3 else 0
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda")
    g.manual_seed(4242)
    w = torch.randn((N, K), generator=g, device="cuda", dtype=torch.float32) * 0.02
    for _ in range(2):
        blocks = rq.quantize_weights(w, type_, wgroup)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(3, args.steps // 4)
    e0.record()
    for _ in range(reps):
        blocks = rq.quantize_weights(w, type_, wgroup)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    # CPU: the reference's own code where it was compiled here (no weight-group modes there), else the port
    sample = min(N, 256)
    ws = w[:sample].cpu().numpy()
    if oracle.have_ref() and wgroup == 0:
        cpu, kind = oracle.Ref(), "reference"
        fn = lambda: cpu.quantize_weights(ws, type_)
    else:
        cpu, kind = oracle.Port(), "port"
        fn = lambda: cpu.quantize_weights(ws, type_, wgroup=wgroup)
    best = float("inf")
    for _ in range(3):
        t0 = time.perf_counter()
        want = fn()
        best = min(best, time.perf_counter() - t0)
    same = bool((blocks[:sample].cpu().numpy() == want).all())
    print(json.dumps({"wquant": {"K": K, "N": N, "type": type_, "wgroup": wgroup}, "ms": ms, "rows_per_s": N / (ms * 1e-3),
                      "GBps_fp32_in": N * K * 4 / (ms * 1e-3) / 1e9,
                      "cpu": {"rows_per_s": sample / best, "cores": os.cpu_count(), "kind": kind, "sample_rows": sample},
                      "bit_identical_on_sample": same}))


def time_shape(K, N, M, type_, path, G, steps, warmup, copies=0, probe=True):
    """One shape: a CUDA graph of back-to-back matmuls over enough distinct weight copies to overflow L2 (the method of
    the reference's own bench, rig/ggml_bench.cpp), whole node, contraction kernel alone, rotate+quantize alone."""
    import torch

    import ruquant_b200 as rq
    from ruquant_b200 import synth

    dev = torch.device("cuda", torch.cuda.current_device())
    wbytes = N * (K // 256) * 144
    copies = copies if copies > 0 else max(1, -(-(384 << 20) // wbytes)) if M <= 64 else 1
    layouts = rq.PREPACK_ALL if path == 0 else (rq.PREPACK_DECODE if path == 1 else rq.PREPACK_PREFILL)
    if path == 0:
        layouts = rq.PREPACK_DECODE if M <= 64 else rq.PREPACK_PREFILL
    base = synth.random_weights(N, K, type_, seed=1, device=dev)
    weights = []
    for c in range(copies):
        blocks = base if c == 0 else torch.roll(base, c, 0).contiguous()
        w = rq.Weight(blocks.view(-1), type_, K, N=N, layouts=layouts)
        w.blocks = None
        weights.append(w)
    del base
    x = torch.randn((M, K), device=dev, dtype=torch.float32)
    y = torch.empty((M, N), device=dev, dtype=torch.float32)
    ws = rq.new_workspace(K, M, dev)
    stream = torch.cuda.Stream(device=dev)

    def node():
        for w in weights:
            rq.mul_mat(w, x, out=y, clip=1.0, act_group=G, path=path, workspace=ws, stream=stream)

    def contraction():
        for w in weights:
            rq.mul_mat_quantized(w, M, ws, out=y, act_group=G, path=path, stream=stream)

    def quant_only():
        for w in weights:
            rq.quantize(x, w.n_rot, 1.0, G, workspace=ws, stream=stream, fmt=rq.act_format(w, M, path))

    def nofold():
        for w in weights:
            rq.tc_nofold_probe(w, M, ws, y, stream=stream)

    def timed(fn):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            fn()
            stream.synchronize()
            with torch.cuda.graph(g, stream=stream):
                fn()
            for _ in range(warmup):
                g.replay()
            stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                g.replay()
            e1.record(stream)
            stream.synchronize()
        return e0.elapsed_time(e1) * 1e3 / steps / copies      # us per matmul

    us_node, us_con, us_q = timed(node), timed(contraction), timed(quant_only)
    us_probe = None
    if probe and layouts & rq.PREPACK_PREFILL and (path == 2 or M > 64):
        with torch.cuda.stream(stream):
            quant_only()              # leave an activation of the right format in the workspace
        us_probe = timed(nofold)
    rq.device_status(ws, K, M)
    hbm_peak, _, kind = measured_peaks()
    ab, ops = algorithmic_bytes(K, N, M), 2.0 * M * N * K
    return {"single": {"K": K, "N": N, "M": M, "type": type_, "group": G, "path": path, "copies": copies},
            "us_node": us_node, "us_contraction": us_con, "us_rotate_quantize": us_q,
            "GBps_node": ab / us_node / 1e3, "GBps_contraction": ab / us_con / 1e3,
            "frac_hbm_node": ab / us_node / 1e3 / hbm_peak, "frac_hbm_contraction": ab / us_con / 1e3 / hbm_peak,
            "TOPS_node": ops / us_node / 1e6, "TOPS_contraction": ops / us_con / 1e6,
            "us_nofold_probe": us_probe, "TOPS_nofold_probe": (ops / us_probe / 1e6) if us_probe else None,
            "peak_kind": "of " + kind}


def run_single(args):
    """K,N,M[,type]: time one shape instead of the stack."""
    import torch
    parts = [int(v) for v in args.single.split(",")]
    K, N, M = parts[:3]
    type_ = parts[3] if len(parts) > 3 else 45
    torch.cuda.set_device(0)
    print(json.dumps(time_shape(K, N, M, type_, args.path, args.group, args.steps, args.warmup, args.copies)))


# the reference's own performance cases for these types (tests/test-backend-ops.cpp hunk in
# patches/llama.cpp-ruquant.patch:3067-3074): (rows, tokens, K)
REF_PERF_SHAPES = [(17408, n, 5120) for n in (1, 8, 16, 512)] + [(5120, n, 17408) for n in (1, 8, 16, 512)] + \
                  [(6144, n, 5120) for n in (1, 8, 16, 512)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-prefill-stack", action="store_true", help="skip the M = 4096 pass over the whole stack")
    ap.add_argument("--replicated-quantizer", action="store_true", help="N > 1 prefill: every rank quantizes all tokens (no exchange of codes)")
    ap.add_argument("--share-threshold", type=int, default=400000,
                    help="N > 1 prefill: ranks share the quantizer where K times the Paley order reaches this")
    ap.add_argument("--no-perf-shapes", action="store_true", help="skip the reference's own performance shapes")
    ap.add_argument("--single", default="", help="K,N,M[,type]: time one shape instead of the stack")
    ap.add_argument("--wquant", default="", help="K,N[,type[,wgroup]]: time the GPU weight quantizer beside the reference's CPU code")
    ap.add_argument("--gather", default="push", choices=["push", "nccl"], help="N > 1: how a layer's output is assembled")
    ap.add_argument("--copies", type=int, default=0)
    ap.add_argument("--group", type=int, default=64)
    ap.add_argument("--path", type=int, default=0)
    args = ap.parse_args()
    if args.wquant:
        run_wquant(args)
    elif args.single:
        run_single(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
