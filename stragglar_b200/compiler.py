"""Python face of the native schedule compiler and host executor.

:func:`compile_table` lowers an algorithm (``stragglar``, ``stragglar_a2a``,
``ring``, ``rhd``, ``direct``, ``rsag``, ``reducescatter``) for ``n`` ranks into
one op table per physical rank; :func:`host_allreduce` runs a table with host
threads over numpy buffers, walking it exactly like the CUDA kernels do.  The
native code lives in ``csrc/core`` and is loaded from
``stragglar_b200/lib/libsar_core.so`` (built on first use when a C++ compiler
is available).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
import threading
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

from .schedule import Schedule

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_HERE)
_LIB_PATH = os.path.join(_HERE, "lib", "libsar_core.so")
_CORE_SOURCES = ["plan.cpp", "host_exec.cpp", "c_api.cpp"]

MAX_RANKS = 16
VER_STRIDE = 32
OP_DTYPE = np.dtype([
    ("kind", "u1"), ("flags", "u1"), ("round", "u1"), ("chunk", "u1"), ("part", "u1"), ("parts", "u1"),
    ("nsrc", "u1"), ("local_ver", "u1"), ("post_ver", "u1"), ("push_ver", "u1"), ("lane", "u1"), ("pad", "u1"),
    ("src", "u1", (MAX_RANKS,)), ("src_ver", "u1", (MAX_RANKS,)),
])
COPY, REDUCE, REDUCE_PUSH, PUSH = 0, 1, 2, 3
F_SCALE, F_LOCAL = 1, 2
DTYPES = {"float32": 0, "bfloat16": 1, "float16": 2}
ALGORITHMS = ("stragglar", "stragglar_a2a", "ring", "rhd", "direct", "rsag", "reducescatter")

_lock = threading.Lock()
_lib = None


def build_core(force: bool = False) -> str:
    """Compile ``csrc/core`` into ``libsar_core.so`` (host code only)."""
    srcs = [os.path.join(_ROOT, "csrc", "core", s) for s in _CORE_SOURCES]
    deps = srcs + [os.path.join(_ROOT, "csrc", "core", h) for h in
                   ("plan.h", "table.h", "host_exec.h", "c_api.h", "builtin_schedules.inc")]
    if not force and os.path.exists(_LIB_PATH):
        if all(os.path.getmtime(_LIB_PATH) >= os.path.getmtime(d) for d in deps if os.path.exists(d)):
            return _LIB_PATH
    os.makedirs(os.path.dirname(_LIB_PATH), exist_ok=True)
    tmp = _LIB_PATH + f".{os.getpid()}.tmp"
    subprocess.check_call(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-pthread", *srcs, "-o", tmp])
    os.replace(tmp, _LIB_PATH)
    return _LIB_PATH


def lib():
    global _lib
    with _lock:
        if _lib is None:
            if all(os.path.exists(os.path.join(_ROOT, "csrc", "core", s)) for s in _CORE_SOURCES):
                build_core()
            L = C.CDLL(_LIB_PATH)
            L.sar_program_build.restype = C.c_void_p
            L.sar_program_build.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_char_p, C.c_char_p, C.c_int]
            L.sar_program_free.argtypes = [C.c_void_p]
            L.sar_program_num_phases.restype, L.sar_program_num_phases.argtypes = C.c_int, [C.c_void_p]
            L.sar_program_phase.restype, L.sar_program_phase.argtypes = C.c_void_p, [C.c_void_p, C.c_int]
            L.sar_table_participants.restype, L.sar_table_participants.argtypes = C.c_uint32, [C.c_void_p]
            L.sar_host_execute_program.restype = C.c_uint32
            L.sar_host_execute_program.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_uint64, C.c_int, C.c_uint32,
                                                   C.c_float, C.c_int, C.POINTER(C.c_double), C.c_double]
            for name in ("nranks", "num_chunks", "num_rounds", "max_version", "channel", "blocks_hint", "stages_hint", "gate_rounds", "lane1_eighths"):
                f = getattr(L, f"sar_table_{name}")
                f.restype, f.argtypes = C.c_int, [C.c_void_p]
            for name in ("num_ops", "num_round_begin"):
                f = getattr(L, f"sar_table_{name}")
                f.restype, f.argtypes = C.c_int, [C.c_void_p, C.c_int]
            L.sar_table_ops.restype, L.sar_table_ops.argtypes = C.c_void_p, [C.c_void_p, C.c_int]
            L.sar_table_round_begin.restype, L.sar_table_round_begin.argtypes = C.c_void_p, [C.c_void_p, C.c_int]
            for name in ("chunks_in", "chunks_out"):
                f = getattr(L, f"sar_table_{name}")
                f.restype, f.argtypes = C.c_double, [C.c_void_p, C.c_int]
            L.sar_pick_tile_elems.restype = C.c_uint32
            L.sar_pick_tile_elems.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]
            L.sar_host_execute.restype = C.c_uint32
            L.sar_host_execute.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_uint64, C.c_int, C.c_uint32,
                                           C.c_float, C.c_int, C.POINTER(C.c_double), C.c_double, C.c_int]
            L.sar_status_string.restype, L.sar_status_string.argtypes = C.c_char_p, [C.c_uint32]
            _lib = L
    return _lib


class CompileError(ValueError):
    pass


@dataclass
class RankTable:
    rank: int
    ops: np.ndarray          # structured array of OP_DTYPE
    round_begin: np.ndarray  # uint16 offsets into ops, one more than the number of rounds
    chunks_in: float         # chunks this rank pulls from or has pushed by peers (roofline input)
    chunks_out: float


class Table:
    """One compiled phase: a :class:`RankTable` per physical rank.  Owned by
    its :class:`Program`."""

    def final_versions(self, rank: int):
        """Per chunk, the version rank ``rank``'s slot has when the collective is done (how often the slot is
        rewritten): what a staged launch waits for before it copies a tile back to the caller's tensor."""
        out = (C.c_uint8 * 16)()
        lib().sar_table_final_ver(self._h, rank, out)
        return [int(v) for v in out[: self.num_chunks]]

    def __init__(self, handle: int, program: "Program"):
        L = lib()
        self._h = handle
        self._program = program   # keeps the native object alive
        self.n = L.sar_table_nranks(handle)
        self.num_chunks = L.sar_table_num_chunks(handle)
        self.num_rounds = L.sar_table_num_rounds(handle)
        self.max_version = L.sar_table_max_version(handle)
        self.channel = L.sar_table_channel(handle)
        self.blocks_hint = L.sar_table_blocks_hint(handle)
        self.stages_hint = L.sar_table_stages_hint(handle)         # bulk-copy path: ring stages per block (0: all)
        self.gate_rounds = bool(L.sar_table_gate_rounds(handle))   # rounds run one after the other (STRAGGLAR_GATE)
        self.lane1_eighths = L.sar_table_lane1_eighths(handle)     # share of the blocks of lane 1 (4: half)
        self.participants = L.sar_table_participants(handle)
        L.sar_table_final_ver.restype, L.sar_table_final_ver.argtypes = None, [C.c_void_p, C.c_int, C.POINTER(C.c_uint8)]
        self.ranks: List[RankTable] = []
        for r in range(self.n):
            k = L.sar_table_num_ops(handle, r)
            if k:
                raw = C.string_at(L.sar_table_ops(handle, r), k * OP_DTYPE.itemsize)
                ops = np.frombuffer(raw, dtype=OP_DTYPE).copy()
            else:
                ops = np.zeros(0, dtype=OP_DTYPE)
            nb = L.sar_table_num_round_begin(handle, r)
            rb = np.frombuffer(C.string_at(L.sar_table_round_begin(handle, r), 2 * nb), dtype=np.uint16).copy() \
                if nb else np.zeros(1, dtype=np.uint16)
            self.ranks.append(RankTable(r, ops, rb, L.sar_table_chunks_in(handle, r), L.sar_table_chunks_out(handle, r)))

    def takes_part(self, rank: int) -> bool:
        return bool(self.participants >> rank & 1)

    def link_chunks(self) -> float:
        """Largest per-rank traffic in one direction, in chunks: the NVLink
        roofline of the phase is ``link_chunks * chunk_bytes / bandwidth``."""
        return max(max(r.chunks_in, r.chunks_out) for r in self.ranks) if self.ranks else 0.0


class Program:
    """A collective as it is launched: one phase, or two for ``direct`` with
    its pre-phase (the non-stragglers' all-reduce on channel 1, then all ranks
    on channel 0)."""

    def __init__(self, handle: int, alg: str, n: int, prephase: bool, straggler: Optional[int]):
        L = lib()
        self._h = handle
        self.alg, self.n, self.prephase, self.straggler = alg, n, prephase, straggler
        self.phases: List[Table] = [Table(L.sar_program_phase(handle, i), self)
                                    for i in range(L.sar_program_num_phases(handle))]

    def __del__(self):
        try:
            if self._h:
                lib().sar_program_free(self._h)
                self._h = None
        except Exception:
            pass

    @property
    def main(self) -> Table:
        return self.phases[-1]

    @property
    def num_rounds(self) -> int:
        return sum(t.num_rounds for t in self.phases)

    def link_bytes(self, nbytes: int) -> float:
        """Bytes the busiest rank moves in one direction for a buffer of ``nbytes``."""
        return sum(t.link_chunks() * nbytes / t.num_chunks for t in self.phases)


def compile_program(alg: str, n: int, prephase: bool = True, straggler: Optional[int] = None,
                    schedule: Optional[Schedule] = None) -> Program:
    """Compile ``alg`` for ``n`` ranks.  ``prephase=False`` means the caller has
    already run the pre-phase among the n-1 non-stragglers (the bench's
    DELAY = -1 mode).  ``straggler`` names the physical rank that plays logical
    rank n-1 (default: rank n-1 itself).  ``schedule`` overrides the built-in
    StragglAR schedule."""
    L = lib()
    err = C.create_string_buffer(512)
    text = schedule.format(footer=False).encode() if schedule is not None else None
    h = L.sar_program_build(alg.encode(), n, int(prephase), -1 if straggler is None else straggler, text, err, 512)
    if not h:
        raise CompileError(err.value.decode())
    return Program(h, alg, n, prephase, straggler)


def compile_table(alg: str, n: int, prephase: bool = True, straggler: Optional[int] = None,
                  schedule: Optional[Schedule] = None) -> Table:
    """Single-phase convenience around :func:`compile_program`."""
    prog = compile_program(alg, n, prephase, straggler, schedule)
    if len(prog.phases) != 1:
        raise CompileError(f"{alg} with its pre-phase has {len(prog.phases)} phases; use compile_program")
    return prog.phases[0]


def pick_tile_elems(count: int, esize: int, num_chunks: int, blocks: int, min_bytes: int = 4096,
                    max_bytes: int = 131072) -> int:
    return lib().sar_pick_tile_elems(count, esize, num_chunks, blocks, min_bytes, max_bytes)


def gate_min_bytes() -> int:
    """Buffers of at least this many bytes run a gated table with round gating (STRAGGLAR_GATE_MIN_BYTES)."""
    f = lib().sar_gate_min_bytes
    f.restype = C.c_uint64
    return int(f())


def status_string(code: int) -> str:
    return lib().sar_status_string(code).decode()


def host_allreduce(table, bufs: Sequence[np.ndarray], scale: float = 1.0, blocks: int = 2,
                   tile_elems: int = 0, delay_ms: Optional[Sequence[float]] = None, timeout_s: float = 20.0,
                   repeats: int = 1) -> int:
    """Run a :class:`Table` or :class:`Program` in place over ``bufs`` (one
    contiguous array per rank, all of one dtype and length) with ``blocks``
    host threads per rank.  Returns the status code (0 = ok)."""
    n = table.n
    if len(bufs) != n:
        raise ValueError(f"need {n} buffers")
    dt = bufs[0].dtype
    if dt == np.float32:
        code = 0
    elif dt == np.float16:
        code = 2
    elif dt == np.uint16:   # bfloat16 bit patterns
        code = 1
    else:
        raise TypeError(f"unsupported dtype {dt}")
    for b in bufs:
        if b.dtype != dt or b.size != bufs[0].size or not b.flags.c_contiguous or not b.flags.writeable:
            raise ValueError("buffers must be contiguous, writable, same dtype and size")
    ptrs = (C.c_void_p * n)(*[b.ctypes.data for b in bufs])
    dl = (C.c_double * n)(*delay_ms) if delay_ms is not None else None
    if isinstance(table, Program):
        return lib().sar_host_execute_program(table._h, ptrs, bufs[0].size, code, tile_elems, scale, blocks, dl,
                                              timeout_s)
    return lib().sar_host_execute(table._h, ptrs, bufs[0].size, code, tile_elems, scale, blocks, dl, timeout_s, repeats)


_KIND_NAMES = {COPY: "copy", REDUCE: "reduce", REDUCE_PUSH: "match", PUSH: "push"}


def describe(program: Program) -> str:
    """Human-readable listing of a compiled program: per phase and rank, one
    line per op (round, lane, kind, chunk and tile range, peers, versions)."""
    out = []
    for pi, t in enumerate(program.phases):
        out.append(f"phase {pi}: channel {t.channel}, {t.num_chunks} chunks, {t.num_rounds} rounds, "
                   f"participants {[r for r in range(t.n) if t.takes_part(r)]}, "
                   f"link traffic {t.link_chunks():g} chunks per direction on the busiest rank"
                   + (f", at most {t.blocks_hint} blocks per rank" if t.blocks_hint else "")
                   + (", rounds gated" if t.gate_rounds else ""))
        for r in t.ranks:
            if not len(r.ops):
                continue
            out.append(f"  rank {r.rank}: in {r.chunks_in:g} / out {r.chunks_out:g} chunks")
            for o in r.ops:
                kind, n = int(o["kind"]), int(o["nsrc"])
                peers = [int(x) for x in o["src"][:n]]
                vers = [int(x) for x in o["src_ver"][:n]]
                part = "" if int(o["parts"]) == 1 else f" part {int(o['part']) + 1}/{int(o['parts'])}"
                flags = ("+scale" if int(o["flags"]) & F_SCALE else "") + ("+own" if int(o["flags"]) & F_LOCAL else "")
                arrow = "->" if kind == PUSH else "<-"
                out.append(f"    round {int(o['round']):2d} lane {int(o['lane'])} {_KIND_NAMES[kind]:6s} chunk {int(o['chunk']):2d}{part} "
                           f"{arrow} {peers} (needs v{vers}, own v{int(o['local_ver'])}) => own v{int(o['post_ver'])}"
                           + (f", peer v{int(o['push_ver'])}" if kind in (PUSH, REDUCE_PUSH) else "") + (f" {flags}" if flags else ""))
    return "\n".join(out)


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(description="compile a collective and list its per-rank op tables")
    ap.add_argument("alg", choices=ALGORITHMS)
    ap.add_argument("n", type=int)
    ap.add_argument("--no-prephase", action="store_true", help="the pre-phase has already happened (DELAY = -1)")
    ap.add_argument("--straggler", type=int, default=None, help="physical rank that plays logical rank n-1")
    ap.add_argument("--schedule", default=None, help="file with a synthesizer printout to use instead of the built-in schedule")
    args = ap.parse_args(argv)
    sched = Schedule.parse(open(args.schedule).read()) if args.schedule else None
    try:
        prog = compile_program(args.alg, args.n, not args.no_prephase, args.straggler, sched)
    except CompileError as e:
        print(f"error: {e}")
        return 1
    print(describe(prog))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
