#!/usr/bin/env python
"""Benchmark of the quantized matrix product on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--m M] [--workload c2|c1|c3...] [--impl reference]

A step is one matmul of the workload's weight matrix with one batch of M
synthetic token rows.  The default workload is the prefill GEMM the headline
metric is quoted on: Q4_K W[17408, 5120] (0.02*N(0,1), quantized by the
library's own quantizer) times bf16 X[M=2048, 5120] (rows of N(0,1) at RMS 1),
fp32 accumulate; `--workload c1` is the decode GEMV.  With --gpus N the weight
rows are split over the ranks (one process per GPU, total work fixed: strong
scaling) and, inside the timed step, every rank's product stores its rows of
the result into every rank's copy of a shared output from its epilogue (plain
stores over NVLink) and a barrier kernel closes the exchange; `--exchange
nccl` does the same with an NCCL all-gather after the product, `--exchange
none` leaves a rank's rows on the rank.

One JSON line is printed by rank 0.  `value` is measured with inputs resident
in HBM; `e2e` goes through the public API from pinned host memory and back;
`parity` compares the output that was timed with the CPU oracle on sampled
rows, on every rank.  `--impl reference` times the CPU restatement of the
reference's own path (oracle/, all host threads) on a bounded sample of the
same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (format, rows, cols, default M, activation dtype)
    "c1": ("q4_k", 17408, 5120, 1, "f32"),      # decode GEMV, f32 activations
    "c2": ("q4_k", 17408, 5120, 2048, "bf16"),  # prefill GEMM, bf16 activations
    "c2_down": ("q4_k", 5120, 17408, 2048, "bf16"),
    "c3_q6k": ("q6_k", 151936, 5120, 1, "f32"),
    "c3_q8": ("q8_0", 5120, 5120, 1, "f32"),
    "c3_attn": ("q4_k", 12288, 5120, 1, "f32"),
    # the feed-forward block gate/up [17408,5120], down [5120,17408], tensor parallel over the ranks
    "c5": ("q4_k", 17408, 5120, 1, "bf16"),
    # every matrix product of one decoded token: 64 layers + the vocabulary head (rows/cols here: the FFN's)
    "c4": ("q4_k", 17408, 5120, 1, "f32"),
}
L2_BYTES = 126 * 1024 * 1024


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p["bf16_tflops"], "tflops_sustained": p.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi sampled every 200 ms while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.path = index, None, None

    def __enter__(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=f, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if not self.path or not os.path.exists(self.path):
            return out
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            f = [s.strip() for s in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            busy = sorted(sm)[len(sm) // 2:]          # the upper half: samples under load
            out.update(sm_mhz=statistics.median(busy), sm_max_mhz=max(mx), samples=len(sm), reasons=sorted(reasons))
        return out


def make_inputs(fmt, rows, cols, m, act, seed_w=0, seed_x=2):
    """W ~ 0.02*N(0,1) f32 (quantized later, on the device); X rows ~ N(0,1)
    (scaled to RMS 1 and rounded to bf16 for the bf16 workloads)."""
    w = 0.02 * np.random.default_rng(seed_w).standard_normal((rows, cols), dtype=np.float32)
    x = np.random.default_rng(seed_x).standard_normal((m, cols), dtype=np.float32)
    if act == "bf16":
        x /= np.sqrt((x * x).mean(1, keepdims=True))
        bits = ((x.view(np.uint32) + 0x7FFF + ((x.view(np.uint32) >> 16) & 1)) >> 16).astype(np.uint16)  # RNE
        x = (bits.astype(np.uint32) << 16).view(np.float32)
        return w, x, bits
    return w, x, None


def algorithmic_bytes(fmt, rows, cols, m):
    from dwim_b200 import row_bytes
    return rows * row_bytes(fmt, cols) + m * cols * 4 + m * rows * 4


# ---------------------------------------------------------------------------------------
# weights of one decoder pass (config 4) over the weights of one [17408, 5120] matrix:
# 64 x 3 FFN matrices + 16 x (12288 + 2 x 1024 + 6144) + 48 x (10240 + 6144 + 6144) rows of 5120,
# and the Q6_K head counted by its bytes (210 against 144 per block)
DECODER_OVER_FFN_MATRIX = (64 * 3 * 17408 + 16 * (12288 + 2048 + 6144) + 48 * (10240 + 6144 + 6144) + 151936 * 210 / 144) / 17408


def run_reference(args, fmt, rows, cols, m, act, ffn=False, decoder=False):
    """The reference's CPU path (restated in oracle/) on the host cores.  For the
    feed-forward block: one [rows, cols] product timed, times three (gate, up and
    down hold the same number of weights; the SiLU is noise beside them)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    oracle.build()
    cores = oracle.threads()
    w, x, _ = make_inputs(fmt, min(rows, 4096), cols, m, act)
    blocks_all = oracle.quantize(fmt, w)
    rb = oracle.row_bytes(fmt, cols)
    # size the sample so that a step takes about a second
    probe_rows = min(w.shape[0], max(cores * 4, 64))
    t = time.perf_counter()
    oracle.matmul(fmt, blocks_all[: probe_rows * rb], probe_rows, cols, x[: min(m, 16)])
    per_row_token = (time.perf_counter() - t) / (probe_rows * min(m, 16))
    sample_rows = int(max(cores, min(w.shape[0], rows, 1.0 / max(per_row_token * m, 1e-12))))
    sample_rows = max(cores, sample_rows // cores * cores)
    blocks = blocks_all[: sample_rows * rb]
    for _ in range(max(1, args.warmup // 3)):
        oracle.matmul(fmt, blocks, sample_rows, cols, x)
    t = time.perf_counter()
    for _ in range(args.steps):
        oracle.matmul(fmt, blocks, sample_rows, cols, x)
    dt = (time.perf_counter() - t) / args.steps
    full = dt * rows / sample_rows                       # a whole step, scaled by rows
    metric, unit, value = headline(fmt, rows, cols, m, full)
    sample = f"{sample_rows} of {rows} weight rows x {m} tokens per step, time scaled by rows"
    if ffn:
        full *= 3
        metric, unit, value = "q4k_ffn_tok_per_s", "tok/s", m / full
        sample += ", times three for gate, up and down"
    if decoder:
        full *= DECODER_OVER_FFN_MATRIX
        metric, unit, value = "decode_matmul_tok_per_s", "tok/s", m / full
        sample += f", times {DECODER_OVER_FFN_MATRIX:.1f} for the weights of the whole pass"
    print(json.dumps({
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": full * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": (ffn_config(rows, cols, m, act, args.gpus) if ffn else
                   {"workload": f"all matrix products of one decoder pass, {m} token(s): 64 layers Q4_K + Q6_K head", "tokens": m}
                   if decoder else workload_config(fmt, rows, cols, m, act, args.gpus, args.exchange)),
        "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "tok_per_s": m / full,
    }))


def timed_e2e(step, n_steps):
    """(median, mean) seconds of a step that ends with a blocking copy to the
    host: the median, because one stall of the host among twenty steps would
    otherwise decide the number."""
    times = []
    for i in range(n_steps):
        t0 = time.perf_counter()
        step(i)
        times.append(time.perf_counter() - t0)
    return statistics.median(times), sum(times) / len(times)


def headline(fmt, rows, cols, m, seconds):
    """The metric of a step: TFLOP/s for the GEMM sizes, GB/s for the GEMV sizes."""
    if m > 16:
        return "q4k_prefill_gemm_tflops" if fmt == "q4_k" else f"{fmt}_gemm_tflops", "TFLOP/s", 2.0 * m * rows * cols / seconds / 1e12
    return ("q4k_decode_gemv_hbm_gbs" if fmt == "q4_k" else f"{fmt}_gemv_hbm_gbs"), "GB/s", algorithmic_bytes(fmt, rows, cols, m) / seconds / 1e9


LINK_GBS = 770.0   # measured peer copy per direction on this pool's NVLink 5 (900 nominal)


def workload_config(fmt, rows, cols, m, act, gpus, exchange="none"):
    if gpus > 1:
        sharding = {
            "push": (f"rows/{gpus}; every rank's product stores its rows of the f32 result into all {gpus} copies of a shared "
                     "output from its epilogue (TMA stores from shared memory over NVLink, while other tiles multiply), then one barrier "
                     "kernel: the all-gather is inside the timed step"),
            "nccl": f"rows/{gpus} + NCCL all-gather of the f32 result + re-assembly kernel, inside the timed step",
            "none": (f"rows/{gpus}; a rank's rows of the result stay on it (they are the K slice its part of the "
                     "down projection multiplies): no exchange in the step"),
        }[exchange]
    else:
        sharding = "none"
    return {"workload": f"{fmt.upper()} W[{rows},{cols}] x {act} X[{m},{cols}], fp32 accumulate",
            "format": fmt, "rows": rows, "cols": cols, "tokens": m, "activations": act,
            "sharding": sharding, "exchange": exchange if gpus > 1 else "none",
            "l2": "weights rotate over copies totalling more than the 126 MB L2"}


def conftest_max_rel_err(got, want) -> float:
    """max |got - want| / max(|want|, rms(want)), the parity tests' measure."""
    got, want = np.asarray(got, np.float64).ravel(), np.asarray(want, np.float64).ravel()
    rms = np.sqrt(np.mean(want * want)) if want.size else 0.0
    den = np.maximum(np.abs(want), max(rms, 1e-30))
    return float(np.max(np.abs(got - want) / den)) if want.size else 0.0


def parity_of(fmt, cols, x, got_rows, w_rows):
    """The timed output against the oracle on sampled weight rows, all tokens.
    `got_rows` is [tokens, sample], `w_rows` the f32 weights of the sampled rows
    (the oracle quantizes them itself: the device quantizer is byte-exact with it)."""
    import oracle
    oracle.build()
    blocks = oracle.quantize(fmt, w_rows)
    want = oracle.matmul(fmt, blocks, w_rows.shape[0], cols, x)
    return conftest_max_rel_err(got_rows, want)


# ---------------------------------------------------------------------------------------
def run_gpu(args, name, fmt, rows, cols, m, act, quiet=False, act_f16=False):
    import torch
    from dwim_b200 import B200, Tensor, shard_rows

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = B200(local)
    if act_f16:
        dev.activation_precision("f16")
    ext = torch.cuda.ExternalStream(dev.stream, device=local)

    w, x, bits = make_inputs(fmt, rows, cols, m, act)
    align = 16
    r0, r1 = shard_rows(rows, rank, world, align)
    my_rows = r1 - r0
    part_rows = shard_rows(rows, 0, world, align)[1]
    t_w = dev.quantize(fmt, w[r0:r1])
    # rotate over enough copies of the weights that a pass cannot be served from L2
    wbytes = max(t_w.data.size, 1)
    copies = int(min(16, max(2, -(-3 * L2_BYTES // wbytes))))
    weights = [dev.upload(t_w) for _ in range(copies)]

    xb = dev.alloc(m * cols)
    (dev.write_bf16(xb, bits) if bits is not None else dev.write(xb, x))
    exchange = args.exchange if world > 1 else "none"
    outs = []
    if exchange == "push":
        # two shared results, alternating: a rank may run one step ahead of its peers
        for _ in range(2):
            buf, handle = dev.shared_alloc(m * rows)
            handles = [None] * world
            dist.all_gather_object(handles, handle)
            dev.shared_connect(buf, world, rank, handles)
            outs.append(buf)
        dist.barrier()
    elif exchange == "nccl":
        if my_rows != part_rows:
            raise SystemExit(f"{rows} rows do not split evenly over {world} ranks at multiples of {align}")
        with torch.cuda.stream(ext):
            parts_t = torch.empty(world * m * part_rows, dtype=torch.float32, device=f"cuda:{local}")
        mine_t = parts_t[rank * m * part_rows:(rank + 1) * m * part_rows]
        out_local = dev.wrap(mine_t.data_ptr(), m * my_rows)
        parts = dev.wrap(parts_t.data_ptr(), parts_t.numel())
        outs.append(dev.alloc(m * rows))
    else:
        outs.append(dev.alloc(m * my_rows))

    per_rank = []

    def product(i):
        if exchange == "push":
            out = outs[i % 2]
            dev.matmul_gather(out, weights[i % copies], xb, r0, rows)
            dev.shared_barrier(out)
        elif exchange == "nccl":
            dev.matmul(out_local, weights[i % copies], xb)
            with torch.cuda.stream(ext):
                dist.all_gather_into_tensor(parts_t, mine_t)
            dev.gather_rows(outs[0], parts, m, rows, world, align)
        else:
            dev.matmul(outs[0], weights[i % copies], xb)

    def step(i, fresh_input=True):
        if fresh_input:
            # the input counts as rewritten (by a bf16 producer where the workload's activations are bf16):
            # its 16-bit operand form is rebuilt inside the step
            (dev.touch_bf16(xb) if bits is not None else dev.touch(xb))
        product(i)

    def timed(n_steps, fresh_input=True):
        if dist:
            dist.barrier()
        torch.cuda.synchronize()
        dev.sync()
        launches0 = dev.launches
        h0 = time.perf_counter()
        dev.timer_begin()
        for i in range(n_steps):
            step(i, fresh_input)
        issue_ms = (time.perf_counter() - h0) * 1e3
        ms = dev.timer_end()
        per_rank.clear()
        per_rank.append({"device_ms_per_step": ms / n_steps, "host_issue_ms_per_step": issue_ms / n_steps})
        if world > 1:
            torch.cuda.synchronize()
            dist.barrier()
            t = torch.tensor([ms, issue_ms], device="cuda")
            all_t = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(all_t, t)
            per_rank.clear()
            per_rank.extend({"device_ms_per_step": float(v[0]) / n_steps, "host_issue_ms_per_step": float(v[1]) / n_steps} for v in all_t)
            ms = max(float(v[0]) for v in all_t)
        return ms / 1e3, dev.launches - launches0

    for i in range(max(args.warmup, 3)):
        step(i)
    with ClockSampler(local) as clocks:
        seconds, launches = timed(args.steps)
        ranks_report = list(per_rank)
        # the dominant kernel alone (operand form cached, no exchange): what the roofline is about
        saved = exchange
        kernel_seconds = None
        if exchange == "none":
            kernel_seconds, _ = timed(args.steps, fresh_input=False)
    per_step = seconds / args.steps
    if kernel_seconds is None:
        # N > 1 with an exchange: the product alone on this rank's rows, into a local buffer
        local_out = dev.alloc(m * my_rows)
        dev.sync()
        for i in range(3):
            dev.matmul(local_out, weights[i % copies], xb)
        dev.timer_begin()
        for i in range(args.steps):
            dev.matmul(local_out, weights[i % copies], xb)
        kernel_seconds = dev.timer_end() / 1e3
        del local_out
    per_kernel = kernel_seconds / args.steps
    metric, unit, value = headline(fmt, rows, cols, m, per_step)

    # ---- a long timed region: clocks settle under sustained load (the short one above runs in the boost window) ----
    sustained = None
    if args.sustain > 0 and not quiet:
        n_long = int(max(args.steps, min(200000, args.sustain / max(per_step, 1e-6))))
        with ClockSampler(local) as long_clocks:
            long_s, _ = timed(n_long)
        _, _, long_value = headline(fmt, rows, cols, m, long_s / n_long)
        sustained = {"value": long_value, "unit": unit, "steps": n_long, "seconds": long_s, "ms_per_step": long_s / n_long * 1e3,
                     "clocks": long_clocks.summary()}

    # ---- parity of what was just timed: sampled weight rows, every token, against the oracle ----
    (dev.touch_bf16(xb) if bits is not None else dev.touch(xb))
    product(0)
    product(1)                                       # both shared results, when there are two
    dev.sync()
    if dist:
        dist.barrier()
    rng = np.random.default_rng(1234 + rank)
    worst, sampled = 0.0, 0
    for out in outs:
        got = dev.read(out)
        if exchange == "none":
            sample = np.unique(np.concatenate([np.arange(min(my_rows, 130)), np.arange(max(0, my_rows - 130), my_rows),
                                               rng.choice(my_rows, min(my_rows, 128), replace=False)]))
            got_rows, w_rows = got.reshape(m, my_rows)[:, sample], w[r0:r1][sample]
        else:
            # the assembled result on this rank: rows from every rank's shard, the cuts included
            cuts = np.concatenate([np.arange(max(0, b - 8), min(rows, b + 8)) for b in
                                   (shard_rows(rows, r, world, align)[0] for r in range(world))])
            sample = np.unique(np.concatenate([cuts, np.arange(rows - 64, rows), rng.choice(rows, min(rows, 320), replace=False)]))
            got_rows, w_rows = got.reshape(m, rows)[:, sample], w[sample]
        tok = np.arange(m) if m <= 256 else np.unique(np.concatenate([np.arange(130), np.arange(m - 130, m), rng.choice(m, 64, replace=False)]))
        worst = max(worst, parity_of(fmt, cols, x[tok], got_rows[tok], w_rows))
        sampled = int(sample.size)
        n_tok = int(tok.size)
        del got
    del w
    if dist:
        t = torch.tensor([worst], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        worst = float(t.item())
    parity = {"max_rel_err": worst, "tolerance": 1e-3, "ok": bool(worst <= 1e-3), "rows_sampled_per_rank": sampled,
              "tokens_checked": n_tok, "checked": "every rank's copy of the timed output against the CPU oracle"
              if exchange != "none" else "every rank's rows of the timed output against the CPU oracle"}

    # ---- end to end: pinned host memory -> device -> product -> pinned host memory ----
    if bits is not None:
        hx = torch.empty(m * cols, dtype=torch.uint16, pin_memory=True).numpy()
        hx[:] = bits.ravel()
    else:
        hx = torch.empty(m * cols, dtype=torch.float32, pin_memory=True).numpy()
        hx[:] = x.ravel()
    hout = torch.empty(len(outs[0]), dtype=torch.float32, pin_memory=True).numpy()
    e2e_steps = max(3, min(args.steps, 20))

    def e2e_step(i):
        (dev.write_bf16(xb, hx) if bits is not None else dev.write(xb, hx))
        product(i)
        dev.read(outs[i % len(outs)], hout)

    # Large batches go in chunks of 256 tokens over three contexts of the device (a context is a
    # stream; weight handles are valid on all of them), one host thread each: the copy in of one
    # chunk, the product of another and the copy out of a third overlap, as an engine that feeds
    # a long prompt would issue them.
    e2e_note = "median over the steps, each timed on the host from the copy in to the copy out"
    lanes = []
    if exchange == "none" and m >= 512:
        from concurrent.futures import ThreadPoolExecutor
        chunk, n_lanes = 256, 3
        for k in range(n_lanes):
            d = dev if k == 0 else B200(local)
            if act_f16 and k:
                d.activation_precision("f16")
            lanes.append((d, d.alloc(chunk * cols), d.alloc(chunk * my_rows)))
        pool = ThreadPoolExecutor(n_lanes)

        def lane_work(k, i):
            d, xc, oc = lanes[k]
            for c in range(k, -(-m // chunk), n_lanes):
                t0, nt = c * chunk, min(chunk, m - c * chunk)
                d.resize(xc, nt * cols)
                d.resize(oc, nt * my_rows)
                src = hx[t0 * cols:(t0 + nt) * cols]
                (d.write_bf16(xc, src) if bits is not None else d.write(xc, src))
                d.matmul(oc, weights[i % copies], xc)
                d.read(oc, hout[t0 * my_rows:(t0 + nt) * my_rows])

        def e2e_step(i):   # noqa: F811 - the pipelined form replaces the plain one
            for f in [pool.submit(lane_work, k, i) for k in range(n_lanes)]:
                f.result()
        e2e_note = ("median over the steps, each timed on the host from the first copy in to the last copy out; the batch goes "
                    "in chunks of 256 tokens over three contexts (streams) of the device, so copies and products overlap")

    for i in range(2):
        e2e_step(i)
    if lanes:
        # the chunked result is the whole result
        chunked = hout.copy()
        dev.matmul(outs[0], weights[1 % copies], xb)
        assert np.array_equal(chunked, dev.read(outs[0])), "the chunked end-to-end result differs from the whole batch's"
    if dist:
        dist.barrier()
    e2e_s, e2e_mean_s = timed_e2e(e2e_step, e2e_steps)
    if lanes:
        pool.shutdown()
        for d, xc, oc in lanes[1:]:
            del xc, oc
        lanes_devs = [d for d, _, _ in lanes[1:]]
        lanes.clear()
        for d in lanes_devs:
            d.close()
    if world > 1:
        t = torch.tensor([e2e_s, e2e_mean_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s, e2e_mean_s = float(t[0].item()), float(t[1].item())
    _, _, e2e_value = headline(fmt, rows, cols, m, e2e_s)

    line = None
    if rank == 0:
        pk = peaks()
        gemm = m > 16
        # DRAM bytes per launch of the dominant kernel from the ncu captures summarised under
        # profiles/ (dram__bytes_read.sum + dram__bytes_write.sum); None where no capture exists.
        traffic, traffic_note = None, None
        if world == 1 and (fmt, rows, cols) == ("q4_k", 17408, 5120):
            if m == 1:
                traffic, traffic_note = 50.48e6, "profiles/dwim_smallm_kernel_q4k_c1.md"
            elif gemm:
                # captured at M=512; weights fixed, operand reads in proportion to M, output in full
                traffic = 50.1e6 + (10.6e6 + 35.65e6) * m / 512
                traffic_note = ("profiles/gemm_q4k_kernel_c2.md: reads captured at M=512 (weights once + 10.6 MB of "
                                "operands per 512 tokens) scaled by M, plus the output in full")
        if gemm:
            flops = 2.0 * m * my_rows * cols
            achieved = flops / per_kernel / 1e12
            roof = {"bound": "tensor", "achieved": achieved, "peak": pk["tflops"], "unit": "TFLOP/s",
                    "frac": achieved / pk["tflops"], "traffic": traffic, "traffic_source": traffic_note,
                    "peak_source": pk["source"],
                    "frac_of_sustained": achieved / pk["tflops_sustained"] if pk["tflops_sustained"] else None,
                    "frac_of_nominal_2250": achieved / 2250.0}
        else:
            by = algorithmic_bytes(fmt, my_rows, cols, m)
            achieved = by / per_kernel / 1e9
            roof = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / pk["hbm_gbs"], "traffic": traffic, "traffic_source": traffic_note,
                    "peak_source": pk["source"],
                    "frac_of_nominal_8tbs": achieved / 8000.0}
        roof["kernel_us"] = per_kernel * 1e6
        if exchange != "none":
            # the fused step: no faster than the slower of its product at the measured peak and its
            # bytes over NVLink at the measured per-direction rate
            link_bytes = (world - 1) * m * my_rows * 4
            t_link = link_bytes / (LINK_GBS * 1e9)
            t_math = (2.0 * m * my_rows * cols / (pk["tflops"] * 1e12)) if gemm else algorithmic_bytes(fmt, my_rows, cols, m) / (pk["hbm_gbs"] * 1e9)
            roof["step"] = {"bound": "nvlink" if t_link > t_math else roof["bound"], "target_us": max(t_link, t_math) * 1e6,
                            "achieved_us": per_step * 1e6, "frac": max(t_link, t_math) / per_step,
                            "nvlink_bytes_out_per_rank": int(link_bytes), "nvlink_gbs_out_per_rank": link_bytes / per_step / 1e9,
                            "nvlink_peak_gbs": LINK_GBS, "nvlink_frac": link_bytes / per_step / 1e9 / LINK_GBS}
        line = {
            "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 (exact integer weights x f16 activations), f32 accumulate", "data": "synthetic",
            "config": workload_config(fmt, rows, cols, m, act, world, exchange),
            "tok_per_s": m / per_step,
            "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": int(hx.nbytes),
                    "d2h_bytes_per_step": int(hout.nbytes), "ms_per_step": e2e_s * 1e3, "ms_per_step_mean": e2e_mean_s * 1e3,
                    "note": e2e_note},
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "roofline": roof,
            "parity": parity,
            "device": dev.name(),
            "ranks": ranks_report,
        }
        if sustained:
            if gemm and pk["tflops_sustained"]:
                sustained["frac_of_sustained_peak"] = sustained["value"] / world / pk["tflops_sustained"]
            line["sustained"] = sustained
    # release everything before another workload runs in this process
    del weights, outs
    dev.close()
    return line


def ffn_config(inner, hidden, m, act, gpus):
    return {"workload": f"feed-forward block: Q4_K gate, up [{inner},{hidden}], down [{hidden},{inner}] x {act} X[{m},{hidden}]",
            "format": "q4_k", "rows": inner, "cols": hidden, "tokens": m, "activations": act,
            "sharding": (f"tensor parallel over {gpus}: gate/up by rows, down by the same K blocks (cuts at multiples of "
                         "256), the f32 [tokens, hidden] partial sums added over the ranks (see reduction)") if gpus > 1 else "none",
            "l2": "blocks rotate over copies totalling more than the 126 MB L2"}


def run_ffn(args, fmt, inner, hidden, m, act):
    """Config 5: out = down . (silu(gate . x) * (up . x)), tokens per second."""
    import torch
    from dwim_b200 import B200, Tensor, shard

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = B200(local)

    # every rank draws the same block (seed 5) and keeps its shard
    rng = np.random.default_rng(5)
    b, e = shard.ffn_cuts(inner, world)[rank]
    full = []                                   # rank 0 keeps the whole block for the parity check
    def quantized(rows, cols, keep_rows=None, keep_cols=None):
        w = 0.02 * rng.standard_normal((rows, cols), dtype=np.float32)
        if rank == 0:
            full.append(w)
        if keep_rows is not None:
            w = w[keep_rows[0]:keep_rows[1]]
        if keep_cols is not None:
            w = np.ascontiguousarray(w[:, keep_cols[0]:keep_cols[1]])
        return dev.quantize(fmt, w) if w.shape[0] and w.shape[1] else None
    gate, up, down = quantized(inner, hidden, (b, e)), quantized(inner, hidden, (b, e)), quantized(hidden, inner, None, (b, e))
    my_inner = e - b
    if not my_inner:
        raise SystemExit(f"rank {rank} of {world} holds no part of the block")
    my_bytes = gate.data.size + up.data.size + down.data.size
    copies = int(min(24, max(2, -(-3 * L2_BYTES // my_bytes))))
    push = world > 1 and args.exchange == "push"
    blocks = [shard.ShardedFFN(dev, gate, up, down, 0, 1, exchange="push" if push else "nccl") for _ in range(copies)]   # already this rank's shard
    # --exchange nccl: the partial sums through NCCL, or for a few tokens through the library's small all-reduce
    peer, reduction = None, "NCCL all-reduce"
    if push:
        reduction = ("fused: the down projection's epilogue stores partial sums into their rows' owners, the owners add "
                     "and store the sums into every rank's copy (two barrier kernels, no collective call)")
    elif world > 1 and m * hidden <= 16 * 1024 and not args.nccl:   # measured: at 8 tokens (160 KB) NCCL is level with it
        try:
            peer = shard.PeerReduce(dev, rank, world, 16 * 1024)
            reduction = "peer-store all-reduce (library kernel over IPC-mapped mailboxes)"
        except Exception as exc:   # noqa: BLE001 - NCCL takes over
            reduction = f"NCCL all-reduce (peer set-up failed: {exc!r})"[:200]
    for blk in blocks:
        blk.world, blk.rank, blk.peer = world, rank, peer
    x = np.random.default_rng(6).standard_normal((m, hidden), dtype=np.float32)
    bits = None
    if act == "bf16":
        x /= np.sqrt((x * x).mean(1, keepdims=True))
        bits = ((x.view(np.uint32) + 0x7FFF + ((x.view(np.uint32) >> 16) & 1)) >> 16).astype(np.uint16)
    xb = dev.alloc(m * hidden)
    (dev.write_bf16(xb, bits) if bits is not None else dev.write(xb, x))

    def step(i):
        (dev.touch_bf16(xb) if bits is not None else dev.touch(xb))   # the input counts as rewritten: its operand form is rebuilt
        return blocks[i % copies].forward(xb)

    def timed(n_steps):
        if dist:
            dist.barrier()
        torch.cuda.synchronize()
        dev.sync()
        launches0 = dev.launches
        dev.timer_begin()
        for i in range(n_steps):
            step(i)
        ms = dev.timer_end()
        if world > 1:
            torch.cuda.synchronize()
            dist.barrier()
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / 1e3, dev.launches - launches0

    for i in range(max(args.warmup, 3)):
        step(i)
    with ClockSampler(local) as clocks:
        seconds, launches = timed(args.steps)
    per_step = seconds / args.steps

    # parity of what was timed: a sample of tokens through the oracle's whole block on rank 0,
    # against every rank's result
    (dev.touch_bf16(xb) if bits is not None else dev.touch(xb))
    got = dev.read(blocks[0].forward(xb)).reshape(m, hidden)
    tok = np.arange(m) if m <= 24 else np.unique(np.concatenate([np.arange(8), np.arange(m - 8, m), np.random.default_rng(9).choice(m, 8, replace=False)]))
    xs = ((bits.astype(np.uint32) << 16).view(np.float32) if bits is not None else x).reshape(m, hidden)[tok]
    want_t = torch.zeros(tok.size * hidden, dtype=torch.float32, device="cuda")
    if rank == 0:
        import oracle
        oracle.build()
        # (the device quantizer's bytes: byte-exact with the oracle's, and much faster on 267 M weights)
        qg, qu, qd = (dev.quantize(fmt, w).data for w in full)
        hmid = oracle.swiglu(fmt, qg, qu, inner, hidden, xs)
        want_t.copy_(torch.from_numpy(oracle.matmul(fmt, qd, hidden, inner, hmid).ravel()))
        del qg, qu, qd
    full.clear()
    if dist:
        dist.broadcast(want_t, 0)
    worst = conftest_max_rel_err(got[tok], want_t.cpu().numpy())
    if dist:
        t = torch.tensor([worst], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        worst = float(t.item())
    parity = {"max_rel_err": worst, "tolerance": 1e-3, "ok": bool(worst <= 1e-3), "tokens_checked": int(tok.size),
              "checked": "every rank's copy of the block's output, all rows, against the CPU oracle's whole block"}

    # end to end: pinned host x -> device -> block -> pinned host out
    hx = torch.empty(m * hidden, dtype=torch.uint16 if bits is not None else torch.float32, pin_memory=True).numpy()
    hx[:] = (bits if bits is not None else x).ravel()
    hout = torch.empty(m * hidden, dtype=torch.float32, pin_memory=True).numpy()
    def e2e_step(i):
        (dev.write_bf16(xb, hx) if bits is not None else dev.write(xb, hx))
        dev.read(blocks[i % copies].forward(xb), hout)
    e2e_steps = max(3, min(args.steps, 20))
    for i in range(2):
        e2e_step(i)
    if dist:
        dist.barrier()
    e2e_s, _ = timed_e2e(e2e_step, e2e_steps)
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())

    line = None
    if rank == 0:
        pk = peaks()
        if m > 16:
            achieved = 2.0 * m * 3 * my_inner * hidden / per_step / 1e12
            roof = {"bound": "tensor", "achieved": achieved, "peak": pk["tflops"], "unit": "TFLOP/s",
                    "frac": achieved / pk["tflops"], "traffic": None, "peak_source": pk["source"]}
        else:
            achieved = (my_bytes + m * hidden * 8 + m * my_inner * 8) / per_step / 1e9
            roof = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / pk["hbm_gbs"], "traffic": None, "peak_source": pk["source"]}
        roof["note"] = "the whole step on this rank (three products, prologues, all-reduce), not one kernel"
        line = {
            "metric": "q4k_ffn_tok_per_s", "value": m / per_step, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16/int8 (exact integer weights), f32 accumulate", "data": "synthetic",
            "config": dict(ffn_config(inner, hidden, m, act, world), reduction=reduction if world > 1 else "none"),
            "e2e": {"value": m / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": int(hx.nbytes),
                    "d2h_bytes_per_step": int(hout.nbytes), "ms_per_step": e2e_s * 1e3},
            "gpu_launches": int(launches), "clocks": clocks.summary(), "roofline": roof, "parity": parity, "device": dev.name(),
        }
        if world == 1 and not args.no_cpu_baseline:
            cb = cpu_baseline(fmt, inner, hidden, m, act)
            dt = cb["ms_per_step"] * 3 / 1e3
            line["cpu_baseline"] = {"value": m / dt, "unit": "tok/s", "cores": cb["cores"], "kind": "port",
                                    "sample": cb["sample"] + ", times three for gate, up and down", "ms_per_step": dt * 1e3}
        return line
    return None


def run_decoder(args, m):
    """Config 4: the matrix products of one decoder pass over m tokens, in the
    engine's order (inference/qwen35/mod.rs:547-654; shapes and call counts after
    gpu/tests.rs:431-436, 476-600): 16 attention layers (q+gate [12288,5120], k
    and v [1024,5120], o [5120,6144]), 48 linear-attention layers (qkv
    [10240,5120], z [6144,5120], out [5120,6144]), each followed by the
    feed-forward block (gate, up [17408,5120], down [5120,17408]) in Q4_K, and
    the vocabulary head [151936,5120] in Q6_K.  Every layer has its own copy of
    its weights in HBM (14.4 GB in all), so L2 cannot help.  What sits between
    the products (norms, attention, rope, ...) is not on this path and not run;
    an input counts as rewritten wherever the engine would have rewritten it."""
    import torch
    from dwim_b200 import B200, row_bytes, shard, shard_rows

    # N > 1: tensor parallel.  Products whose output feeds a per-head or per-row step (q, k, v, qkv,
    # z, gate, up, the head) are split by rows and their results stay on the rank; the two that
    # close a sub-layer (o / out and down) are split along K the same way and their partial sums
    # are added over the ranks: two reductions per layer, through the library's all-reduce over
    # peer memory while they are small (NCCL otherwise).
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = B200(local)
    rng = np.random.default_rng(4)
    hidden, inner, attn, vocab = 5120, 17408, 6144, 151936

    def host(fmt, rows, cols):
        return dev.quantize(fmt, 0.02 * rng.standard_normal((rows, cols), dtype=np.float32))
    span = lambda n, align: (lambda be: be[1] - be[0])(shard_rows(n, rank, world, align))
    my_inner, my_attn, my_vocab = span(inner, 256), span(attn, 256), span(vocab, 16)
    shapes = {"qg": (span(12288, 16), hidden), "kv": (span(1024, 16), hidden), "o": (hidden, my_attn), "qkv": (span(10240, 16), hidden),
              "z": (my_attn, hidden), "gate": (my_inner, hidden), "down": (hidden, my_inner)}
    proto = {k: host("q4_k", *v) for k, v in shapes.items()}
    head = dev.upload(host("q6_k", my_vocab, hidden))
    layers, total = [], my_vocab * row_bytes("q6_k", hidden)
    for l in range(64):
        names = ["qg", "kv", "kv", "o"] if l % 4 == 3 else ["qkv", "z", "o"]
        names += ["gate", "gate", "down"]
        layers.append([dev.upload(proto[n]) for n in names])
        total += sum(proto[n].data.size for n in names)
    x = dev.buffer(rng.standard_normal((m, hidden), dtype=np.float32))        # the residual stream's normalized copy
    a = dev.buffer(rng.standard_normal((m, my_attn), dtype=np.float32))       # this rank's heads' attention output
    outs = {k: dev.alloc(m * shapes[k][0]) for k in ("qg", "kv", "qkv", "z")}
    h, scratch, logits = dev.alloc(m * my_inner), dev.alloc(m * my_inner), dev.alloc(m * my_vocab)
    part_t = torch.zeros(m * hidden, dtype=torch.float32, device="cuda")      # a closing product's result / partial sums
    part = dev.wrap(part_t.data_ptr(), m * hidden)
    ext = torch.cuda.ExternalStream(dev.stream)
    peer, reduction = None, "none"
    if world > 1:
        reduction = "NCCL all-reduce"
        if m * hidden <= 16 * 1024 and not args.nccl:
            try:
                peer = shard.PeerReduce(dev, rank, world, 16 * 1024)
                reduction = "peer-store all-reduce (library kernel over IPC-mapped mailboxes)"
            except Exception as exc:   # noqa: BLE001 - NCCL takes over
                reduction = f"NCCL all-reduce (peer set-up failed: {exc!r})"[:200]

    def closing(w, src):
        """o / out and down: on one GPU the engine's matmul_add into the residual stream;
        tensor parallel the rank's partial product, summed over the ranks."""
        if world == 1:
            dev.matmul_add(part, w, src)
        else:
            dev.matmul(part, w, src)
            reduce_part()

    def reduce_part():
        if peer is not None:
            peer(part, m * hidden)
        else:
            with torch.cuda.stream(ext):
                dist.all_reduce(part_t)

    def token():
        for l, w in enumerate(layers):
            dev.touch(x)                                    # the layer's normalized input
            if l % 4 == 3:
                dev.matmul(outs["qg"], w[0], x); dev.matmul(outs["kv"], w[1], x); dev.matmul(outs["kv"], w[2], x)
                dev.touch(a); closing(w[3], a)
                f = w[4:]
            else:
                dev.matmul(outs["qkv"], w[0], x); dev.matmul(outs["z"], w[1], x)
                dev.touch(a); closing(w[2], a)
                f = w[3:]
            dev.touch(x)                                    # normalized again before the feed-forward block
            dev.swiglu(h, f[0], f[1], x, scratch)
            closing(f[2], h)
        dev.touch(x)
        dev.matmul(logits, head, x)

    for _ in range(max(2, args.warmup // 2)):
        token()
    dev.sync()
    steps = max(3, min(args.steps, 20))
    with ClockSampler(local) as clocks:
        if dist:
            torch.cuda.synchronize()
            dist.barrier()
        launches0 = dev.launches
        dev.timer_begin()
        for _ in range(steps):
            token()
        seconds = dev.timer_end() / 1e3 / steps
        launches = (dev.launches - launches0) // steps
        if dist:
            torch.cuda.synchronize()
            t = torch.tensor([seconds], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            seconds = float(t.item())
    # the same pass replayed as one CUDA graph (captured from the library's stream; everything
    # it allocates lazily exists by now): what is left of the time when the host issues nothing
    graph = None
    try:
        if world > 1:
            raise RuntimeError("one GPU only: the reductions are not captured")
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=ext):
            token()
        with torch.cuda.stream(ext):
            for _ in range(2):
                g.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                g.replay()
            e1.record()
        torch.cuda.synchronize()
        gs = e0.elapsed_time(e1) / 1e3 / steps
        graph = {"value": m / gs, "unit": "tok/s", "ms_per_step": gs * 1e3}
    except Exception as exc:   # noqa: BLE001 - reported in the line, the eager number stands
        graph = {"unavailable": repr(exc)[:200]}
    dev.sync()
    # end to end: the token's embedding row in, the logits out
    hx = torch.empty(m * hidden, dtype=torch.float32, pin_memory=True).numpy(); hx[:] = 0.5
    hl = torch.empty(m * my_vocab, dtype=torch.float32, pin_memory=True).numpy()
    def e2e():
        dev.write(x, hx); token(); dev.read(logits, hl)
    e2e()
    if dist:
        dist.barrier()
    e2e_s, _ = timed_e2e(lambda i: e2e(), 5)
    if dist:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    pk = peaks()
    achieved = total / seconds / 1e9
    if rank != 0:
        return None
    return {
        "metric": "decode_matmul_tok_per_s", "value": m / seconds, "unit": "tok/s", "n_gpus": world, "steps": steps,
        "warmup": max(2, args.warmup // 2), "ms_per_step": seconds * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8/f16 (exact integer weights), f32 accumulate", "data": "synthetic",
        "config": {"workload": f"all matrix products of one decoder pass, {m} token(s): 64 layers Q4_K + Q6_K head, "
                               f"{total / 1e9:.2f} GB of weights resident, each read once per pass",
                   "tokens": m, "products_per_pass": 16 * 7 + 48 * 6 + 1, "l2": "every layer has its own weights in HBM",
                   "sharding": (f"tensor parallel over {world}: q/k/v-type products, gate/up and the head by rows, o/out and down "
                                f"along K; two reductions per layer: {reduction}; weight GB are this rank's") if world > 1 else "none"},
        "e2e": {"value": m / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": int(hx.nbytes), "d2h_bytes_per_step": int(hl.nbytes),
                "ms_per_step": e2e_s * 1e3},
        "gpu_launches": int(launches), "clocks": clocks.summary(), "graph_replay": graph,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                     "traffic": None, "peak_source": pk["source"],
                     "note": "weight bytes of the whole pass over its time: all kernels, prologues and launch gaps included"},
        "device": dev.name(),
    }


def reference_gpu_table(rows, cols, tokens=(1, 16, 128, 512, 2048)):
    """The reference engine's own CUDA kernel on this GPU (matmul_tile.cu, compiled from
    its sources into oracle/_ref/; its host side restated in oracle/ref_gpu.py): Q4_0
    W[rows, cols], which has Q4_K's density, at the same token counts, timed the same
    way (CUDA events, weights rotating over copies beyond L2, warm-up first)."""
    import torch
    import oracle
    from oracle import ref_gpu
    if not ref_gpu.available():
        return {"unavailable": "oracle/_ref/dwim_tile.cubin has not been built"}
    try:
        oracle.build()
        ref = ref_gpu.RefTile()
        rng = np.random.default_rng(0)
        sample = 1024                                            # distinct rows; the matrix repeats them (timing needs no more)
        w = 0.02 * rng.standard_normal((sample, cols), dtype=np.float32)
        scales, quants = ref_gpu.quantize_q4_0(w)
        reps = -(-rows // sample)
        scales, quants = np.tile(scales, (reps, 1))[:rows], np.tile(quants, (reps, 1, 1))[:rows]
        tiled, tiled_scales = ref_gpu.tile_q4_0(scales, quants)
        wbytes = rows * (cols // 2 + 2 * (cols // 32))            # as the reference counts them, gpu/tests.rs:281-293
        copies = int(max(2, -(-3 * L2_BYTES // wbytes)))
        d_w = [torch.from_numpy(tiled.view(np.int32)).cuda() for _ in range(copies)]
        d_s = [torch.from_numpy(tiled_scales.view(np.int16)).cuda() for _ in range(copies)]
        stream = torch.cuda.current_stream().cuda_stream
        table = {}
        for m in tokens:
            x = rng.standard_normal((m, cols), dtype=np.float32)
            d_x = torch.from_numpy(oracle.to_f16(x).view(np.int16)).cuda()
            out = torch.zeros(m * rows, dtype=torch.float32, device="cuda")
            if m == tokens[0]:
                # the harness computes what the reference's CPU path computes: a few rows, every token
                ref.matmul(out.data_ptr(), d_w[0].data_ptr(), d_s[0].data_ptr(), d_x.data_ptr(), rows, cols, m, stream)
                torch.cuda.synchronize()
                got = out.cpu().numpy().reshape(m, rows)
                rows_checked = [0, 1, 127, 128, sample - 1, rows - 1]
                want = np.array([[oracle.dot_q4_0_split(scales[r], quants[r].reshape(-1), x[t]) for r in rows_checked] for t in range(m)])
                typical = float(np.sqrt(np.mean(want * want)))
                check = float(np.abs(got[:, rows_checked] - want).max() / typical)
            steps = 20 if m <= 512 else 8
            for i in range(3):
                ref.matmul(out.data_ptr(), d_w[i % copies].data_ptr(), d_s[i % copies].data_ptr(), d_x.data_ptr(), rows, cols, m, stream)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(steps):
                ref.matmul(out.data_ptr(), d_w[i % copies].data_ptr(), d_s[i % copies].data_ptr(), d_x.data_ptr(), rows, cols, m, stream)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / steps
            table[f"m{m}"] = {"us": us, "weight_gbs": wbytes / us / 1e3, "tflops": 2.0 * m * rows * cols / us / 1e6}
        return {"kernel": "matmul_tile64_q4_0 / matmul_tile16_q4_0 (mma.sync m16n8k16, cp.async, compiled for sm_100)",
                "workload": f"Q4_0 W[{rows},{cols}] x f16 X[M,{cols}], f32 out", "worst_error_over_typical": check, "by_tokens": table}
    except Exception as exc:   # noqa: BLE001 - a baseline that cannot run is reported, the benchmark's own line stands
        return {"unavailable": repr(exc)[:300]}


def cpu_baseline(fmt, rows, cols, m, act):
    """The oracle's matmul on the host cores, on a bounded sample (about 10 s)."""
    import oracle
    oracle.build()
    cores = oracle.threads()
    sample_w = min(rows, 2048)
    w, x, _ = make_inputs(fmt, sample_w, cols, m, act)
    blocks = oracle.quantize(fmt, w)
    rb = oracle.row_bytes(fmt, cols)
    probe = min(sample_w, max(4 * cores, 64))
    t = time.perf_counter()
    oracle.matmul(fmt, blocks[: probe * rb], probe, cols, x[: min(m, 8)])
    unit_s = (time.perf_counter() - t) / (probe * min(m, 8))
    sample_rows = int(min(sample_w, max(cores, 10.0 / max(unit_s * m, 1e-12))))
    t = time.perf_counter()
    reps = 0
    while True:
        oracle.matmul(fmt, blocks[: sample_rows * rb], sample_rows, cols, x)
        reps += 1
        if time.perf_counter() - t > 8.0 or reps >= 200:
            break
    dt = (time.perf_counter() - t) / reps * rows / sample_rows
    _, unit, value = headline(fmt, rows, cols, m, dt)
    return {"value": value, "unit": unit, "cores": cores, "kind": "port",
            "sample": f"{sample_rows} of {rows} rows x {m} tokens, {reps} repeats, time scaled by rows",
            "ms_per_step": dt * 1e3}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--m", "--tokens", dest="m", type=int, default=None, help="tokens per step (default: the workload's)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--nccl", action="store_true", help="c5, N > 1: NCCL for the partial sums even for a few tokens")
    ap.add_argument("--exchange", default="push", choices=["push", "nccl", "none"],
                    help="N > 1: how the row-sharded result reaches every rank inside the step: stores from the product's "
                         "epilogue into every rank's copy (push, default), an NCCL all-gather, or not at all (rows stay sharded)")
    ap.add_argument("--sustain", type=float, default=2.0, help="seconds of the second, long timed region (0: skip)")
    ap.add_argument("--no-also", action="store_true", help="N = 1, default workload: skip the decode GEMV line embedded under 'also'")
    args = ap.parse_args()
    fmt, rows, cols, m, act = WORKLOADS[args.workload]
    if args.m:
        m = args.m
    if args.impl == "reference":
        run_reference(args, fmt, rows, cols, m, act, ffn=args.workload == "c5", decoder=args.workload == "c4")
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world != args.gpus:
        if args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE is {world})")
    if args.workload == "c4":
        line = run_decoder(args, m)
    elif args.workload == "c5":
        line = run_ffn(args, fmt, rows, cols, m, act)
    else:
        line = run_gpu(args, args.workload, fmt, rows, cols, m, act)
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(fmt, rows, cols, m, act)
        if world == 1 and args.workload == "c2" and args.m is None and not args.no_also:
            # the other half of the headline metric, measured in the same process: the decode GEMV
            # (config 1) and every matrix product of a decoded token (config 4)
            also = {}
            f1, r1, c1, m1, a1 = WORKLOADS["c1"]
            l1 = run_gpu(args, "c1", f1, r1, c1, m1, a1, quiet=True)
            also["c1"] = {"metric": l1["metric"], "gbs_per_step": l1["value"], "us_per_step": l1["ms_per_step"] * 1e3,
                          "kernel_us": l1["roofline"]["kernel_us"], "kernel_gbs": l1["roofline"]["achieved"],
                          "frac": l1["roofline"]["frac"], "frac_of_nominal_8tbs": l1["roofline"]["frac_of_nominal_8tbs"],
                          "parity": l1["parity"], "config": l1["config"]["workload"]}
            for tokens in (1, 4):
                l4 = run_decoder(args, tokens)
                also[f"c4_m{tokens}"] = {"metric": l4["metric"], "tok_per_s": l4["value"], "ms_per_pass": l4["ms_per_step"],
                                         "hbm_frac": l4["roofline"]["frac"], "graph_replay": l4["graph_replay"],
                                         "launches_per_pass": l4["gpu_launches"], "config": l4["config"]["workload"]}
            # this library's kernel at the token counts the reference's GPU kernel is raced at
            mine = {}
            for tokens in (16, 128, 512):
                lt = run_gpu(args, "c2", fmt, rows, cols, tokens, act, quiet=True)
                mine[f"m{tokens}"] = {"us": lt["roofline"]["kernel_us"], "step_us": lt["ms_per_step"] * 1e3,
                                      "tflops": 2.0 * tokens * rows * cols / lt["roofline"]["kernel_us"] / 1e6,
                                      "max_rel_err": lt["parity"]["max_rel_err"]}
            # the same product with f32 activations (two f16 columns per token), and the dense kernel's formats
            for key, (f2, r2, c2, a2) in {"c2_f32_activations": (fmt, rows, cols, "f32"), "q8_0_5120x5120": ("q8_0", 5120, 5120, "bf16"),
                                          "q6_k_12288x5120": ("q6_k", 12288, 5120, "bf16")}.items():
                lt = run_gpu(args, "c2", f2, r2, c2, m, a2, quiet=True)
                if key == "c2_f32_activations":
                    # and as one f16 column (dwim_b200_activation_precision: the reference device's precision)
                    l16 = run_gpu(args, "c2", f2, r2, c2, m, a2, quiet=True, act_f16=True)
                    also["c2_f32_activations_as_f16"] = {"tokens": m, "us": l16["roofline"]["kernel_us"], "step_us": l16["ms_per_step"] * 1e3,
                                                         "tflops_per_step": l16["value"], "max_rel_err": l16["parity"]["max_rel_err"],
                                                         "note": "opt-in, the reference device's precision: outside the 1e-3 bar on the worst element by design"}
                also[key] = {"tokens": m, "us": lt["roofline"]["kernel_us"], "step_us": lt["ms_per_step"] * 1e3,
                             "tflops_per_step": lt["value"], "max_rel_err": lt["parity"]["max_rel_err"],
                             "config": lt["config"]["workload"]}
            mine["m1"] = {"us": also["c1"]["kernel_us"], "step_us": also["c1"]["us_per_step"]}
            mine["m2048"] = {"us": line["roofline"]["kernel_us"], "step_us": line["ms_per_step"] * 1e3,
                             "tflops": line["roofline"]["achieved"]}
            also["by_tokens"] = mine
            line["also"] = also
            line["reference_gpu"] = reference_gpu_table(rows, cols)
    if rank == 0 and line is not None:
        print(json.dumps(line))
        sys.stdout.flush()
    if world > 1:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
