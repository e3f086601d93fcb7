"""Tile-level performance model of the table executor.

    python -m stragglar_b200.exec_model stragglar 8 --bytes 1073741824 --blocks 64 [--no-prephase] [--rounds]
    python -m stragglar_b200.exec_model all 8 --bytes 268435456 --no-prephase      # every algorithm, free and gated

The alpha-beta model of :mod:`.simulate` (the reference's stragglar/simulation.py) prices whole rounds.  This
module prices what the persistent kernel actually does: every rank's blocks walk the items of the compiled
table (tile-interleaved within a round, block ``b`` of a lane takes items ``b, b+G, ...``, in order), an item
starts when the flags of its operands are visible, its transfers share the NVLink ports of the two GPUs they
touch max-min fairly (one egress and one ingress port per GPU, as behind an NVSwitch) and are capped per block
by what one block keeps in flight, and its flags become visible to the readers a publication latency after its
last byte.  It answers questions the round model cannot: what a block count or a lane split does to a schedule,
which rank's port is the bottleneck, how much of the time the rounds of a schedule overlap.

It is a fluid model with a fixed time step; no HBM, no SM effects.  The default constants are set from the
measurements on the 8-GPU B200 box (peer copy 770 GB/s per direction, about 64 GB/s per block of the bulk-copy
path, flags visible to a remote poller about 3 us after the last store) and are arguments of :func:`simulate`.
"""
from __future__ import annotations

import argparse
import sys
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np

from . import compiler as sc


@dataclass
class ModelParams:
    link_gbs: float = 770.0        # per GPU and direction
    block_gbs: float = 64.0        # what one block can move (bytes in flight / latency)
    flag_us: float = 3.0           # last byte of a tile -> its flag seen by a reader (fence + store + poll)
    item_us: float = 0.4           # fixed cost per item on the block that runs it
    dt_us: float = 0.25            # time step


@dataclass
class Result:
    time_us: float
    per_rank_us: List[float]
    round_span_us: Dict[int, Tuple[float, float]]         # schedule round -> (first item start, last item done)
    port_busy: Dict[str, List[float]] = field(default_factory=dict)   # "in"/"out" -> busy fraction per rank
    items: int = 0
    timeline_us: float = 0.0                                          # width of a timeline bin
    timeline: Dict[str, np.ndarray] = field(default_factory=dict)     # "in"/"out" -> [bin, rank] port use (0..1)


def _lane_of_block(block: int, nblocks: int, table_lanes: int, lane1_eighths: int = 4):
    """(lanes, lane, position in the lane, blocks of the lane): the rule of sar_lane_of_block (csrc/core/table.h)."""
    lanes = 2 if (table_lanes >= 2 and nblocks >= 2) else 1
    if lanes == 1 or lane1_eighths in (0, 4):
        lane = block % lanes
        return lanes, lane, block // lanes, (nblocks - lane + lanes - 1) // lanes
    n1 = max(1, min(nblocks - 1, (nblocks * min(lane1_eighths, 7) + 4) // 8))
    n0 = nblocks - n1
    return (lanes, 0, block, n0) if block < n0 else (lanes, 1, block - n0, n1)


def _items_of_rank(ops: np.ndarray, num_chunks: int, chunk_tiles: List[int], tile_bytes_of, lanes: int):
    """Per lane, the rank's items in walking order: (op index, chunk, tile, bytes)."""
    out = [[] for _ in range(lanes)]
    rounds = sorted(set(int(r) for r in ops["round"]))
    for rd in rounds:
        idx = [i for i in range(len(ops)) if int(ops["round"][i]) == rd]
        for lane in range(lanes):
            sel = [i for i in idx if (int(ops["lane"][i]) if lanes == 2 else 0) == lane] if lanes == 2 else idx
            if not sel:
                continue
            ranges = []
            for i in sel:
                tiles = chunk_tiles[int(ops["chunk"][i])]
                part, parts = int(ops["part"][i]), max(int(ops["parts"][i]), 1)
                ranges.append((tiles * part // parts, tiles * (part + 1) // parts))
            most = max(t1 - t0 for t0, t1 in ranges)
            for lt in range(most):
                for i, (t0, t1) in zip(sel, ranges):
                    if lt < t1 - t0:
                        c = int(ops["chunk"][i])
                        out[lane].append((i, c, t0 + lt, tile_bytes_of(c, t0 + lt)))
    return out


def simulate(program: sc.Program, nbytes: int, blocks: int = 64, tile_bytes: int = 0,
             params: Optional[ModelParams] = None, phase: int = -1, delay_us: Optional[List[float]] = None,
             timeline_us: float = 0.0, dispatch: str = "static", window: int = 1,
             round_lag: Optional[int] = None) -> Result:
    """Run the model on one phase of ``program`` (default: the last one) for a buffer of ``nbytes`` per rank.
    ``delay_us[r]`` holds rank ``r`` back before its first item.  ``dispatch``: ``"static"`` -- block ``b`` of a
    lane owns the items ``b, b+G, ...`` (what the kernels do); ``"dynamic"`` -- a free block takes the lane's next
    unclaimed item; with ``window > 1`` it takes the first *ready* item among the next ``window`` unclaimed ones
    (and the oldest one when none is ready).  ``round_lag``: ``None`` -- rounds overlap as far as the flags allow;
    ``k`` -- an item of round ``r`` starts only after every rank has finished round ``r - 1 - k`` (0: the rounds run
    one after the other, as in the synchronous model of the schedule)."""
    P = params or ModelParams()
    table = program.phases[phase]
    if round_lag is None and table.gate_rounds and nbytes >= sc.gate_min_bytes():
        round_lag = 0                      # the table is launched with round gating
    n, nch = table.n, table.num_chunks
    if tile_bytes <= 0:   # the tile the library picks for fp32 on the bulk-copy path (at most 64 KiB)
        tile_bytes = 4 * sc.pick_tile_elems(nbytes // 4, 4, nch, blocks, 2048, 65536)
    chunk_bytes = [nbytes // nch + (1 if c < (nbytes % nch) else 0) for c in range(nch)]
    chunk_tiles = [max(1, -(-cb // tile_bytes)) for cb in chunk_bytes]

    def tile_bytes_of(c, t):
        return min(tile_bytes, chunk_bytes[c] - t * tile_bytes)

    # ---- items and their static description
    ready_at: Dict[Tuple[int, int, int, int], float] = {}     # (rank, chunk, tile, version) -> time the flag is visible
    blocks_state = []   # one entry per (rank, lane, block): its item list and position
    ops_of = [table.ranks[r].ops for r in range(n)]
    total_items = 0
    for r in range(n):
        if not table.takes_part(r) or len(ops_of[r]) == 0:
            continue
        table_lanes = 2 if int(ops_of[r]["lane"].max()) > 0 else 1
        lanes = _lane_of_block(0, blocks, table_lanes, table.lane1_eighths)[0]
        per_lane = _items_of_rank(ops_of[r], nch, chunk_tiles, tile_bytes_of, lanes)
        for lane in range(lanes):
            # block 0 is in lane 0 and the last block in lane 1 under both numbering rules
            nb = _lane_of_block(0 if lane == 0 else blocks - 1, blocks, table_lanes, table.lane1_eighths)[3]
            t0 = delay_us[r] if delay_us else 0.0
            if dispatch == "static":
                for b in range(nb):
                    items = per_lane[lane][b::nb]
                    total_items += len(items)
                    if items:
                        blocks_state.append({"rank": r, "items": items, "pos": 0, "state": 0, "t_free": t0, "flows": []})
            else:
                queue = {"items": per_lane[lane], "taken": [False] * len(per_lane[lane]), "head": 0}
                total_items += len(per_lane[lane])
                for b in range(min(nb, len(per_lane[lane]))):
                    blocks_state.append({"rank": r, "items": [None], "pos": 0, "state": 0, "t_free": t0, "flows": [], "queue": queue})
    # items left per schedule round, over all ranks; when a round is complete (and everybody can know it)
    left_in_round: Dict[int, int] = {}
    for B in blocks_state:
        pool = B["queue"]["items"] if "queue" in B else B["items"]
        if "queue" in B and B["queue"].get("counted"):
            continue
        if "queue" in B:
            B["queue"]["counted"] = True
        for it in pool:
            rd = int(ops_of[B["rank"]][it[0]]["round"])
            left_in_round[rd] = left_in_round.get(rd, 0) + 1
    all_rounds = sorted(left_in_round)
    round_done_at: Dict[int, float] = {}

    def round_gate_open(rd: int, t: float) -> bool:
        if round_lag is None:
            return True
        i = all_rounds.index(rd) - 1 - round_lag
        return i < 0 or round_done_at.get(all_rounds[i], np.inf) <= t

    # ---- fluid simulation
    cap = P.link_gbs * 1e3          # bytes per microsecond
    bcap = P.block_gbs * 1e3
    now, dt = 0.0, P.dt_us
    done_blocks = 0
    per_rank = [0.0] * n
    round_span: Dict[int, List[float]] = {}
    busy_in, busy_out = np.zeros(n), np.zeros(n)
    tl_in: List[np.ndarray] = []
    tl_out: List[np.ndarray] = []
    # flows: arrays rebuilt each step from the blocks that are transferring
    steps = 0
    max_steps = int(5e6)
    while done_blocks < len(blocks_state) and steps < max_steps:
        steps += 1
        # 1. blocks that can start their next item
        for B in blocks_state:
            if B["state"] != 0 or B["pos"] >= len(B["items"]) or now < B["t_free"]:
                continue
            r = B["rank"]

            def is_ready(item):
                oi_, c_, t_, _ = item
                op_ = ops_of[r][oi_]
                if not round_gate_open(int(op_["round"]), now):
                    return False
                for q in range(int(op_["nsrc"])):
                    if delay_us and delay_us[int(op_["src"][q])] > now:
                        return False          # the peer has not entered the collective yet (its arrival word)
                    v = int(op_["src_ver"][q])
                    if v and ready_at.get((int(op_["src"][q]), c_, t_, v), np.inf) > now:
                        return False
                lv = int(op_["local_ver"])
                return not (lv and ready_at.get((r, c_, t_, lv), np.inf) > now)

            Q = B.get("queue")
            if Q is not None and B["items"][0] is None:
                # claim an item: the first ready one in the window, else the oldest unclaimed one
                taken, its = Q["taken"], Q["items"]
                while Q["head"] < len(its) and taken[Q["head"]]:
                    Q["head"] += 1
                if Q["head"] >= len(its):
                    B["pos"] = 1
                    done_blocks += 1
                    continue
                cand, seen, pick = Q["head"], 0, Q["head"]
                while cand < len(its) and seen < window:
                    if not taken[cand]:
                        seen += 1
                        if is_ready(its[cand]):
                            pick = cand
                            break
                    cand += 1
                taken[pick] = True
                B["items"][0] = its[pick]
            oi, c, t, nb_ = B["items"][B["pos"]]
            op = ops_of[r][oi]
            kind, nsrc = int(op["kind"]), int(op["nsrc"])
            if not is_ready(B["items"][B["pos"]]):
                continue
            flows = []
            if kind == sc.PUSH:
                flows = [[r, int(op["src"][q]), float(nb_)] for q in range(nsrc)]
            else:
                flows = [[int(op["src"][q]), r, float(nb_)] for q in range(nsrc)]
                if kind == sc.REDUCE_PUSH:
                    flows.append([r, int(op["src"][0]), float(nb_)])
            B["flows"], B["state"] = flows, 1
            rd = int(op["round"])
            span = round_span.setdefault(rd, [now, now])
            span[0] = min(span[0], now)
        # 2. rates: max-min fair over the ports, capped per block
        active = [B for B in blocks_state if B["state"] == 1 and B["flows"]]
        if active:
            src = np.array([f[0] for B in active for f in B["flows"]])
            dst = np.array([f[1] for B in active for f in B["flows"]])
            rem = np.array([f[2] for B in active for f in B["flows"]])
            owner = np.array([i for i, B in enumerate(active) for _ in B["flows"]])
            nfl = len(src)
            per_block_flows = np.bincount(owner, minlength=len(active))
            fcap = bcap / per_block_flows[owner]           # a block's rate is split over its flows
            rate = np.zeros(nfl)
            frozen = np.zeros(nfl, dtype=bool)
            out_left, in_left = np.full(n, cap), np.full(n, cap)
            for _ in range(2 * n + 2):
                live = ~frozen
                if not live.any():
                    break
                cnt_out = np.bincount(src[live], minlength=n).astype(float)
                cnt_in = np.bincount(dst[live], minlength=n).astype(float)
                share_out = np.where(cnt_out > 0, out_left / np.maximum(cnt_out, 1), np.inf)
                share_in = np.where(cnt_in > 0, in_left / np.maximum(cnt_in, 1), np.inf)
                s = np.minimum(share_out[src], share_in[dst])
                s = np.where(live, np.minimum(s, fcap), np.inf)
                m = s.min()
                pick = live & (s <= m * (1 + 1e-9))
                rate[pick] = m if np.isfinite(m) else 0.0
                frozen |= pick
                np.subtract.at(out_left, src[pick], rate[pick])
                np.subtract.at(in_left, dst[pick], rate[pick])
            moved = np.minimum(rem, rate * dt)
            mo, mi = np.bincount(src, weights=moved, minlength=n), np.bincount(dst, weights=moved, minlength=n)
            busy_out += mo
            busy_in += mi
            if timeline_us > 0:
                b = int(now // timeline_us)
                while len(tl_out) <= b:
                    tl_out.append(np.zeros(n)); tl_in.append(np.zeros(n))
                tl_out[b] += mo / (cap * timeline_us)
                tl_in[b] += mi / (cap * timeline_us)
            k = 0
            for B in active:
                for f in B["flows"]:
                    f[2] -= moved[k]
                    k += 1
        now += dt
        # 3. completions
        for B in active:
            if all(f[2] <= 1e-6 for f in B["flows"]):
                r = B["rank"]
                oi, c, t, _ = B["items"][B["pos"]]
                op = ops_of[r][oi]
                kind = int(op["kind"])
                vis = now + P.flag_us
                if kind != sc.PUSH:
                    ready_at[(r, c, t, int(op["post_ver"]))] = vis
                if kind == sc.REDUCE_PUSH:
                    ready_at[(int(op["src"][0]), c, t, int(op["push_ver"]))] = vis
                if kind == sc.PUSH:
                    for q in range(int(op["nsrc"])):
                        ready_at[(int(op["src"][q]), c, t, int(op["push_ver"]))] = vis
                rd = int(op["round"])
                round_span[rd][1] = max(round_span[rd][1], now)
                left_in_round[rd] -= 1
                if left_in_round[rd] == 0:
                    round_done_at[rd] = vis
                B["flows"], B["state"] = [], 0
                B["t_free"] = now + P.item_us
                per_rank[r] = max(per_rank[r], vis)
                if "queue" in B:
                    B["items"][0] = None          # claims the next item when it is free again
                else:
                    B["pos"] += 1
                    if B["pos"] >= len(B["items"]):
                        done_blocks += 1
        # items without any transfer (n = 1) complete at once
        for B in blocks_state:
            if B["state"] == 1 and not B["flows"]:
                B["state"] = 0
                if "queue" in B:
                    B["items"][0] = None
                else:
                    B["pos"] += 1
                    if B["pos"] >= len(B["items"]):
                        done_blocks += 1
    if steps >= max_steps:
        raise RuntimeError("the model did not terminate (a dependency is never satisfied?)")
    total = max(per_rank) if per_rank else 0.0
    return Result(time_us=total, per_rank_us=per_rank,
                  round_span_us={k: (v[0], v[1]) for k, v in sorted(round_span.items())},
                  port_busy={"in": list(busy_in / (cap * max(total, 1e-9))), "out": list(busy_out / (cap * max(total, 1e-9)))},
                  items=total_items, timeline_us=timeline_us,
                  timeline={"in": np.array(tl_in), "out": np.array(tl_out)} if timeline_us > 0 else {})


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="tile-level model of the table executor")
    ap.add_argument("alg")
    ap.add_argument("n", type=int)
    ap.add_argument("--bytes", type=int, default=1 << 28)
    ap.add_argument("--blocks", type=int, default=0, help="blocks per rank (0: the table's hint, else 128)")
    ap.add_argument("--tile-bytes", type=int, default=0, help="0: what the library picks (at most 64 KiB)")
    ap.add_argument("--no-prephase", action="store_true", help="the state after the straggler's arrival (DELAY = -1)")
    ap.add_argument("--straggler", type=int, default=None)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    ap.add_argument("--block-gbs", type=float, default=64.0)
    ap.add_argument("--flag-us", type=float, default=3.0)
    ap.add_argument("--delay-ms", type=float, default=0.0,
                    help="hold the straggler back this long (with the pre-phase in the table: what DELAY > 0 times)")
    ap.add_argument("--rounds", action="store_true", help="print when every schedule round started and ended")
    ap.add_argument("--dispatch", default="static", choices=["static", "dynamic"],
                    help="static: block b owns items b, b+G, ... (the kernels); dynamic: free blocks take the next item")
    ap.add_argument("--window", type=int, default=1, help="dynamic dispatch: look this many items ahead for a ready one")
    ap.add_argument("--round-lag", type=int, default=None,
                    help="an item of round r waits until every rank has finished round r-1-LAG (default: no such gate)")
    ap.add_argument("--timeline", type=float, default=0.0, metavar="US", help="print the port use per rank in bins of US")
    args = ap.parse_args(argv)
    if args.alg == "all":
        # one line per algorithm: free-running rounds and rounds one after the other
        params = ModelParams(link_gbs=args.link_gbs, block_gbs=args.block_gbs, flag_us=args.flag_us)
        print(f"n={args.n}, {args.bytes} bytes per rank; us (fraction of the busiest port's rate)")
        print(f"{'algorithm':14s} {'blocks':>6s} {'free-running':>16s} {'gated rounds':>16s}")
        for alg in ("stragglar", "stragglar_a2a", "ring", "rhd", "rsag", "direct"):
            if alg == "rhd" and args.n & (args.n - 1):
                continue
            try:
                prog = sc.compile_program(alg, args.n, prephase=not args.no_prephase, straggler=args.straggler)
            except RuntimeError as e:
                print(f"{alg:14s} not available: {e}")
                continue
            blocks = args.blocks or (prog.main.blocks_hint if prog.main.blocks_hint > 0 else 128)
            floor = prog.link_bytes(args.bytes) / (args.link_gbs * 1e3)
            free = simulate(prog, args.bytes, blocks, args.tile_bytes, params, round_lag=None if not prog.main.gate_rounds else 10**6)
            gated = simulate(prog, args.bytes, blocks, args.tile_bytes, params, round_lag=0)
            print(f"{alg:14s} {blocks:6d} {free.time_us:9.1f} ({floor / free.time_us:.2f}) {gated.time_us:9.1f} ({floor / gated.time_us:.2f})")
        return 0
    prog = sc.compile_program(args.alg, args.n, prephase=not args.no_prephase, straggler=args.straggler)
    blocks = args.blocks or (prog.main.blocks_hint if prog.main.blocks_hint > 0 else 128)
    delay = None
    if args.delay_ms > 0:
        delay = [0.0] * args.n
        delay[args.straggler if args.straggler is not None else args.n - 1] = args.delay_ms * 1e3
    res = simulate(prog, args.bytes, blocks, args.tile_bytes,
                   ModelParams(link_gbs=args.link_gbs, block_gbs=args.block_gbs, flag_us=args.flag_us), delay_us=delay,
                   timeline_us=args.timeline, dispatch=args.dispatch, window=args.window, round_lag=args.round_lag)
    link = prog.link_bytes(args.bytes) / (args.link_gbs * 1e3)
    if delay:
        print(f"straggler held back {args.delay_ms:g} ms: {res.time_us - args.delay_ms * 1e3:.1f} us after its arrival")
    print(f"{args.alg} n={args.n} {args.bytes} bytes, {blocks} blocks: {res.time_us:.1f} us modelled, "
          f"{link:.1f} us at the busiest port's rate ({link / res.time_us:.2f}), {res.items} items")
    print("port use in:  " + " ".join(f"{x:.2f}" for x in res.port_busy["in"]))
    print("port use out: " + " ".join(f"{x:.2f}" for x in res.port_busy["out"]))
    if args.rounds:
        for rd, (a, b) in res.round_span_us.items():
            print(f"  round {rd:2d}: {a:8.1f} .. {b:8.1f} us")
    if args.timeline > 0:
        for name in ("out", "in"):
            print(f"port use {name} per rank, bins of {args.timeline:g} us:")
            for b, row in enumerate(res.timeline[name]):
                print(f"  {b * args.timeline:7.0f} " + " ".join(f"{x:4.2f}" for x in row))
    return 0


if __name__ == "__main__":
    sys.exit(main())
