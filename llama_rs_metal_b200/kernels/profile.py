"""Per-kernel timing behind a flag: LRM_PROFILE=1.

With the flag set every launch of this library's kernels is bracketed by two
CUDA events on the launching stream, and `report()` (also run at exit) prints
one line per kernel entry point: calls, time, the bytes it has to move and the
floating-point work it has to do, and the fraction of the device's peak that
is (the reference has the same switch, LLAMA_METAL_PROFILE, which times every
dispatch and prints a table, crates/metal-backend/src/apple/commands.rs:187-209).

Under the flag decode steps are not captured in CUDA graphs and no kernel
starts before its predecessor has finished (the events sit between them), so
the times are those of each kernel alone; a whole step is faster than their
sum. A bracketed launch on an idle device also counts the launch's own
start-up: the report measures that floor with an empty-handed kernel and
prints it, and small kernels are to be read against it. Bytes and flops are
what the operation needs by its arguments (every operand once), not what the
hardware moved.
"""
from __future__ import annotations

import atexit
import ctypes
import os
import sys
from typing import Callable, Dict, List, Optional, Tuple

import torch

enabled = os.environ.get("LRM_PROFILE", "0") == "1"

# what the host knows about the step that is running and the kernels cannot tell from their
# arguments: tokens whose keys attention reads, and query-key pairs of a prompt's causal attention
hints: Dict[str, float] = {"kv_tokens": 0, "pairs": 0, "phase": ""}

_ELEM = {0: 4, 1: 2}  # dtype codes of the C entry points -> bytes per element


def _v(a) -> float:
    return getattr(a, "value", a) or 0


def _gemm(M, N, K, out_elem, in_elem=2):
    return in_elem * (M * K + N * K) + out_elem * M * N, 2.0 * M * N * K


def _out_elem(mode) -> int:
    return {0: 2, 1: 4, 2: 8, 3: 1, 4: 4}.get(int(mode), 4)  # add: read and write; gate: half the columns


# entry point -> (bytes, flops) from its positional arguments
WORK: Dict[str, Callable[..., Tuple[float, float]]] = {
    "lrm_embed_rows": lambda a: (_v(a[4]) * _v(a[5]) * (_ELEM[_v(a[1])] + 4), 0),
    "lrm_rms_norm": lambda a: (_v(a[9]) * _v(a[10]) * (4 + _ELEM[_v(a[4])] + 4 * _v(a[7]) + (4 if _v(a[7]) else 0)),
                               3.0 * _v(a[9]) * _v(a[10])),
    "lrm_gemm_f32": lambda a: _gemm(_v(a[3]), _v(a[4]), _v(a[5]), 8 if _v(a[6]) else 4, 4),
    "lrm_gemm_bf16_stream_shaped": lambda a: _gemm(_v(a[3]), _v(a[4]), _v(a[5]), _out_elem(_v(a[6]))),
    "lrm_gemm_bf16_mma": lambda a: _gemm(_v(a[3]), _v(a[4]), _v(a[5]), _out_elem(_v(a[6]))),
    "lrm_gemm_bf16_umma_rows": lambda a: _gemm(_v(a[3]), _v(a[5]), _v(a[6]), _out_elem(_v(a[7]))),
    "lrm_gemm_bf16_umma_pair": lambda a: _gemm(_v(a[3]), _v(a[4]), _v(a[5]), _out_elem(_v(a[6]))),
    # the fused q|k|v projection of a prompt: the product, its bfloat16 result stored packed and k, v again in the cache
    "lrm_gemm_bf16_umma_qkv": lambda a: _gemm(_v(a[2]), _v(a[3]), _v(a[4]), 2),
    "lrm_gemm_bf16_umma_pair_qkv": lambda a: _gemm(_v(a[2]), _v(a[3]), _v(a[4]), 2),
    "lrm_rope_table": lambda a: (_v(a[3]) * _v(a[4]) * 8.0 + _v(a[3]) * 4.0, 0),
    "lrm_gemm_bf16_stream_pick": lambda a: _gemm(_v(a[2]), _v(a[3]), _v(a[4]), 0),
    "lrm_rope_store": lambda a: (2.0 * _v(a[11]) * (_v(a[12]) + 2 * _v(a[13])) * _v(a[14]) * _ELEM[_v(a[1])], 0),
    "lrm_silu_mul": lambda a: (3.0 * _v(a[3]) * _v(a[4]) * _ELEM[_v(a[2])], 0),
    "lrm_add_planes": lambda a: ((_v(a[2]) + 2.0) * _v(a[3]) * 4, 0),
    # prompts: q, k, v, out once; 4 flops per (query, key, head dimension) pair of the causal triangle
    "lrm_attention_prefill_umma": lambda a: (2.0 * _v(a[5]) * 2 * (_v(a[8]) + _v(a[9])) * _v(a[10]),
                                             4.0 * hints["pairs"] * _v(a[8]) * _v(a[10])),
    "lrm_attention_prefill_pingpong": lambda a: (2.0 * _v(a[5]) * 2 * (_v(a[8]) + _v(a[9])) * _v(a[10]),
                                                 4.0 * hints["pairs"] * _v(a[8]) * _v(a[10])),
    "lrm_attention_prefill_tiled": lambda a: (0, 4.0 * hints["pairs"] * _v(a[7]) * _v(a[9])),
    "lrm_attention_packed_rowwise": lambda a: (0, 4.0 * hints["pairs"] * _v(a[8]) * _v(a[10])),
    # over the cache: every cached key and value of the live sequences once
    "lrm_attention_decode_tiled": lambda a: (2.0 * hints["kv_tokens"] * _v(a[11]) * _v(a[12]) * 2, 0),
    "lrm_attention_decode_cluster": lambda a: (2.0 * hints["kv_tokens"] * _v(a[14]) * _v(a[15]) * 2, 0),
    "lrm_attention_paged_rowwise": lambda a: (2.0 * hints["kv_tokens"] * _v(a[13]) * _v(a[14]) * _ELEM[_v(a[4])], 0),
    "lrm_attention_extend_tiled": lambda a: (2.0 * hints["kv_tokens"] * _v(a[12]) * _v(a[13]) * 2,
                                             4.0 * hints["pairs"] * _v(a[11]) * _v(a[13])),
    "lrm_argmax_rows": lambda a: (4.0 * _v(a[4]) * _v(a[5]), 0),
    "lrm_sample_gumbel_rows": lambda a: (4.0 * _v(a[4]) * _v(a[5]), 0),
}
# entry points that only answer questions and launch nothing
_QUERIES = ("_supports", "_slices", "_pieces", "_resident", "_floats", "_error", "_room", "lrm_set_pdl", "lrm_set_norm_ranks", "lrm_pick_pieces")


class _Row:
    __slots__ = ("calls", "events", "bytes", "flops")

    def __init__(self):
        self.calls, self.events, self.bytes, self.flops = 0, [], 0.0, 0.0


_rows: Dict[Tuple[str, str], _Row] = {}  # (entry point, phase of the step that launched it)


class ProfiledLibrary:
    """Stands in for the loaded library: every launching entry point is timed."""

    def __init__(self, lib):
        self._lib = lib

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        if any(q in name for q in _QUERIES):
            return fn

        def timed(*args):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            stream = torch.cuda.current_stream()
            begin.record(stream)
            code = fn(*args)
            end.record(stream)
            row = _rows.setdefault((name, hints["phase"]), _Row())
            row.calls += 1
            row.events.append((begin, end))
            work = WORK.get(name)
            if work is not None:
                try:
                    b, f = work(args)
                    row.bytes += b
                    row.flops += f
                except (IndexError, KeyError, TypeError):
                    pass
            return code
        return timed


def reset() -> None:
    _rows.clear()


def _peaks() -> Tuple[float, float, str]:
    """(GB/s, TFLOP/s, where from): the measured peaks of this machine if a file at the
    repository root gives them, else the figures measured earlier on the same kind of GPU."""
    import json
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as handle:
            data = json.load(handle)
        return float(data["hbm_gbs"]), float(data["bf16_tflops"]), "measured"
    except (OSError, ValueError, KeyError):
        return 6650.0, 1590.0, "fallback"


def table() -> List[dict]:
    """One dict per kernel entry point, slowest first (waits for the device)."""
    torch.cuda.synchronize()
    hbm, tflops, _ = _peaks()
    out = []
    for (name, phase), row in _rows.items():
        ms = sum(b.elapsed_time(e) for b, e in row.events)
        seconds = ms * 1e-3
        gbs = row.bytes / seconds / 1e9 if seconds > 0 else 0.0
        tf = row.flops / seconds / 1e12 if seconds > 0 else 0.0
        out.append(dict(kernel=name, phase=phase, calls=row.calls, ms=ms, us_per_call=ms * 1e3 / max(row.calls, 1),
                        gb_per_s=gbs, tflop_per_s=tf, frac_of_peak=max(gbs / hbm, tf / tflops)))
    return sorted(out, key=lambda r: -r["ms"])


def launch_floor_us() -> float:
    """What a bracketed launch of a kernel with nothing to do takes (median of 20)."""
    from . import library
    lib = getattr(library.load(), "_lib", library.load())
    x = torch.zeros(1, dtype=torch.float32, device="cuda")
    y = torch.zeros(1, dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream()
    raw = ctypes.c_void_p(stream.cuda_stream)
    pairs = []
    for _ in range(20):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record(stream)
        lib.lrm_cast(ctypes.c_void_p(x.data_ptr()), 0, ctypes.c_void_p(y.data_ptr()), 1, ctypes.c_longlong(1), raw)
        end.record(stream)
        pairs.append((begin, end))
    torch.cuda.synchronize()
    times = sorted(b.elapsed_time(e) for b, e in pairs)
    return times[len(times) // 2] * 1e3


def report(file=None) -> None:
    if not _rows:
        return
    file = file or sys.stderr
    rows = table()
    total = sum(r["ms"] for r in rows)
    _, _, source = _peaks()
    print(f"{'kernel':34s} {'phase':8s} {'calls':>7s} {'ms':>9s} {'share':>6s} {'us/call':>9s} {'GB/s':>8s} {'TFLOP/s':>8s} "
          f"{'of peak':>8s}", file=file)
    for r in rows:
        print(f"{r['kernel'][4:]:34s} {r['phase']:8s} {r['calls']:7d} {r['ms']:9.3f} {r['ms'] / total:6.1%} {r['us_per_call']:9.2f} "
              f"{r['gb_per_s']:8.0f} {r['tflop_per_s']:8.1f} {r['frac_of_peak']:8.2f}", file=file)
    print(f"{'total':34s} {'':8s} {sum(r['calls'] for r in rows):7d} {total:9.3f}   (each kernel alone; peaks: {source}; "
          f"a bracketed launch of an empty kernel takes {launch_floor_us():.1f} us)", file=file)


if enabled:
    atexit.register(report)
