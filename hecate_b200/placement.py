"""Routing logs and expert placement for expert parallelism.

The reference records which experts every decode step selects (`EXL3_ROUTE_LOG`, runtime/tier/rtx_graph.py:255-278) and
re-ranks its tiers from those logs (tools/placement/rerank_placement.py). Its tiers are speed classes of one node; here the
"tiers" are the GPUs of an expert-parallel group, and the question the log answers is which experts should share a GPU so
that no GPU gets much more than its share of the picks.

  * `write_route_log` / `read_route_log`: the reference's record format, so logs recorded by either side can be read by
    the other's tools. Header record: u16 0xA55B, u16 n, int16 layer index per slot. Step record: u16 0xA55A, u16 n layers,
    u16 rows, int16 [n][rows][8] placement-local ids.
  * `step_counts`: per layer, in how many steps each expert was selected (distinct per step, as rerank_placement.py counts);
    `pick_counts`: how many picks each expert received (the load of a prefill chunk).
  * `balance`: a placement for `world` GPUs from such counts: experts in descending load, each to the least loaded GPU that
    still has a free slot (every GPU serves the same number of slots, since the kernels take contiguous ranges of equal
    length); optionally the hottest experts are given additional slots on other GPUs and their tokens are dealt out over the
    copies. The result is the `perm` of a placement entry (router position -> expert id) plus, with copies, the table that maps
    (expert, token) to a position.
  * `positions`: applies a plan to a selection (what a router with permuted weight rows would emit directly).
"""
import struct

import numpy as np

TAG_HEADER, TAG_STEP = 0xA55B, 0xA55A


def write_route_log(path, layers, steps, append=False):
    """layers: layer index per slot; steps: iterable of int arrays [n_layers][rows][topk] of placement-local ids."""
    with open(path, "ab" if append else "wb") as f:
        if not append:
            f.write(struct.pack("<HH", TAG_HEADER, len(layers)) + np.asarray(layers, np.int16).tobytes())
        for s in steps:
            s = np.asarray(s)
            n, rows, topk = s.shape
            if n != len(layers) or topk != 8:
                raise ValueError("a step is [n_layers][rows][8]")
            f.write(struct.pack("<HHH", TAG_STEP, n, rows) + s.astype(np.int16).tobytes())


def read_route_log(path):
    """-> (layers, [step arrays int16 [n][rows][8]])."""
    data = open(path, "rb").read()
    off, layers, steps = 0, None, []
    while off + 4 <= len(data):
        tag, n = struct.unpack_from("<HH", data, off)
        if tag == TAG_HEADER:
            if off + 4 + 2 * n > len(data):
                raise ValueError(f"{path}: truncated header record at {off}")
            layers = np.frombuffer(data, np.int16, n, off + 4).tolist(); off += 4 + 2 * n
        elif tag == TAG_STEP:
            if off + 6 > len(data):
                raise ValueError(f"{path}: truncated step record at {off}")
            rows = struct.unpack_from("<H", data, off + 4)[0]
            if off + 6 + 2 * n * rows * 8 > len(data):
                raise ValueError(f"{path}: truncated step record at {off}")
            steps.append(np.frombuffer(data, np.int16, n * rows * 8, off + 6).reshape(n, rows, 8)); off += 6 + 2 * n * rows * 8
        else:
            raise ValueError(f"{path}: bad record tag {tag:#x} at {off}")
    return layers, steps


def step_counts(layers, steps, n_experts=256, perm_by_layer=None):
    """{layer: float64 [n_experts]}: number of steps in which the expert was selected by at least one row. Ids in the log are
    placement-local; perm_by_layer[layer] (position -> expert id) translates them, identity if absent."""
    out = {}
    for i, L in enumerate(layers):
        perm = np.asarray(perm_by_layer[L]) if perm_by_layer and L in perm_by_layer else np.arange(n_experts)
        c = np.zeros(n_experts)
        for s in steps:
            c[perm[np.unique(s[i])]] += 1
        out[L] = c
    return out


def pick_counts(sel, n_experts):
    """int64 [n_experts]: picks per expert in a selection array of any shape."""
    return np.bincount(np.asarray(sel).reshape(-1), minlength=n_experts)[:n_experts].astype(np.int64)


class Plan:
    """perm[p] = expert at router position p (rank r serves positions [r * slots, (r + 1) * slots)); copies[e] = positions of
    expert e (one, or several when it was replicated); load[r] = expected picks of rank r under the counts it was built from."""

    def __init__(self, perm, copies, load, world):
        self.perm, self.copies, self.load, self.world = perm, copies, load, world
        self.slots = len(perm) // world

    def imbalance(self):
        return float(self.load.max() / self.load.mean()) if self.load.mean() > 0 else 1.0

    def table(self):
        """int32 [n_experts][width]: positions of each expert, its list of copies repeated cyclically up to the least common
        multiple of the copy counts (so that token t mod width splits every expert's tokens evenly over its copies)."""
        width = int(np.lcm.reduce([len(c) for c in self.copies]))
        return np.array([[c[i % len(c)] for i in range(width)] for c in self.copies], dtype=np.int32)


def balance(counts, world, extra_slots=0):
    """counts [n_experts] (any non-negative load measure) -> Plan over n_experts + extra_slots positions.

    Every extra slot goes to the expert whose copies currently carry the most load each (its load is then split evenly over
    one more copy); extra_slots must keep the number of positions a multiple of `world`. Copies of one expert are placed on
    different GPUs."""
    counts = np.asarray(counts, dtype=np.float64)
    n = len(counts)
    total = n + extra_slots
    if total % world:
        raise ValueError("experts + extra slots must be a multiple of the world size")
    ncopy = np.ones(n, dtype=np.int64)
    for _ in range(extra_slots):
        per = np.where(ncopy < world, counts / ncopy, -1.0)
        e = int(np.argmax(per))
        if per[e] < 0:
            raise ValueError("more extra slots than copies that fit on different GPUs")
        ncopy[e] += 1
    items = sorted(((counts[e] / ncopy[e], e) for e in range(n) for _ in range(ncopy[e])), key=lambda t: (-t[0], t[1]))
    slots = total // world
    load = np.zeros(world)
    members = [[] for _ in range(world)]
    has = [set() for _ in range(world)]
    for w, e in items:
        order = sorted(range(world), key=lambda r: (load[r], r))
        r = next((r for r in order if len(members[r]) < slots and e not in has[r]), None)
        if r is None:          # only GPUs that already hold a copy have room: accept a second copy there rather than fail
            r = next(r for r in order if len(members[r]) < slots)
        members[r].append(e); has[r].add(e); load[r] += w
    perm = [e for r in range(world) for e in members[r]]
    copies = [[] for _ in range(n)]
    for p, e in enumerate(perm):
        copies[e].append(p)
    return Plan(perm, copies, load, world)


def contiguous(counts, world):
    """The plan of the default placement (expert e at position e), for comparison."""
    counts = np.asarray(counts, dtype=np.float64)
    n = len(counts)
    slots = n // world
    load = np.array([counts[r * slots:(r + 1) * slots].sum() for r in range(world)])
    return Plan(list(range(n)), [[e] for e in range(n)], load, world)


def positions(sel, plan, token_ids=None):
    """Selection in expert ids [rows][topk] -> router positions under `plan`. A replicated expert's tokens are dealt out over
    its copies by token index (token_ids, default the row number)."""
    sel = np.asarray(sel)
    tab = plan.table()
    t = np.arange(sel.shape[0]) if token_ids is None else np.asarray(token_ids)
    return tab[sel, (t % tab.shape[1])[:, None]].astype(sel.dtype)


def permute_router(wt, bias, plan):
    """Router weight rows (and bias) in position order, so that the router emits positions directly. Only for plans without
    copies (a router row cannot stand for two positions)."""
    if any(len(c) != 1 for c in plan.copies):
        raise ValueError("a plan with replicated experts needs positions() after the router")
    idx = np.asarray(plan.perm)
    return wt[idx], (None if bias is None else bias[idx])
