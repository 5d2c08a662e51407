"""Prints the rings, trees and chunk schedules the kernels use.

    python extra/ring_visualize.py --world 8 --nnodes 2 --routes 4

Reads the schedule from the same header the kernels compile (csrc/schedule.h via
libpenny_sim.so), so what is printed is what runs.  For every route it shows the
ring order, each position's peers and the chunk it sends / receives at every
step, and marks inconsistencies: `*` if a position's receive chunk differs from
its predecessor's send chunk, `#` if a chunk is reduced twice or never.  The
reference's extra/ring_visualize.py replays its inter-node ring construction in
Python for 16 PEs and flags the same two conditions.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from penny_b200.parallel import schedule  # noqa: E402

COLORS = ["\033[9%dm" % c for c in (1, 2, 3, 4, 5, 6)] + ["\033[3%dm" % c for c in (1, 2)]
RESET = "\033[0m"


def paint(rank, gpn, text, color):
    return f"{COLORS[(rank // gpn) % len(COLORS)]}{text}{RESET}" if color else text


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--nnodes", type=int, default=1, help="virtual nodes")
    ap.add_argument("--routes", type=int, default=2)
    ap.add_argument("--no-color", action="store_true")
    args = ap.parse_args()
    n, gpn = args.world, args.world // args.nnodes
    color = not args.no_color and sys.stdout.isatty()
    bad = 0
    for route in range(args.routes):
        order = schedule.ring_order(n, args.nnodes, route)
        print(f"route {route}: " + " -> ".join(paint(r, gpn, str(r), color) for r in order) + f" -> {order[0]}")
        counts = [[0] * n for _ in range(n)]
        for pos, r in enumerate(order):
            nxt, prv = order[(pos + 1) % n], order[(pos - 1) % n]
            cells = []
            for step in range(2 * (n - 1)):
                sc, rc, reduce = schedule.ring_step_chunks(n, pos, step)
                psc, _, _ = schedule.ring_step_chunks(n, (pos - 1) % n, step)
                mark = "" if psc == rc else "*"
                if reduce:
                    counts[pos][rc] += 1
                bad += bool(mark)
                cells.append(f"{'R' if reduce else 'G'}{sc}>{rc}{mark}")
            dup = [c for c in range(n) if counts[pos][c] > 1]
            flag = " #" if dup else ""
            bad += bool(dup)
            print(f"  pos {pos} rank {paint(r, gpn, str(r), color)} recv<-{prv} send->{nxt}: " + " ".join(cells) + flag)
    print(f"trees (one per local rank of a {gpn}-GPU node, leaf -> root):")
    for t in range(gpn):
        print(f"  tree {t}: " + " -> ".join(str(x) for x in schedule.tree_chain(gpn, t)))
    print("consistent" if bad == 0 else f"{bad} inconsistencies")
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
