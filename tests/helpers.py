"""Shared helpers of the tests: seeded synthetic layers on the host, their upload, error metrics."""
import numpy as np

from hecate_b200 import synth


class HostLayer:
    """Seeded experts of one layer on the host: packed codes (operator layout) and float32 scales [K/G][N].
    group = 0: one scale per row (the reference's format); 128: the group-quantised benchmark format."""

    def __init__(self, seed, layer, H, I, experts, group, shared=True):
        self.H, self.I, self.group, self.ids = H, I, group, list(experts)
        gh, gi = (group or H), (group or I)
        mk = lambda e: dict(
            gq=synth.packed_codes(seed, layer, "gate_q", e, I, H), uq=synth.packed_codes(seed, layer, "up_q", e, I, H),
            dq=synth.packed_codes(seed, layer, "down_q", e, H, I),
            gs=synth.scales(seed, layer, "gate_s", e, I, H, gh), us=synth.scales(seed, layer, "up_s", e, I, H, gh),
            ds=synth.scales(seed, layer, "down_s", e, H, I, gi))
        self.ex = [mk(e) for e in self.ids]
        self.sh = mk(synth.SHARED) if shared else None

    def oracle_experts(self, O):
        f = lambda d: O.Expert(d["gq"], d["uq"], d["dq"], d["gs"], d["us"], d["ds"], self.H, self.I)
        return [f(d) for d in self.ex], (f(self.sh) if self.sh else None)

    def upload(self, device):
        import torch
        from hecate_b200 import moe
        sdt = torch.float32 if self.group == 0 else torch.bfloat16
        q = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
        from hecate_b200 import layout
        dev_order = (lambda a: a.reshape(-1)) if self.group == 0 else layout.group_scales_device_order
        s = lambda a: torch.from_numpy(np.ascontiguousarray(dev_order(a))).to(device).to(sdt).contiguous()
        cols = {k: [] for k in ("gq", "uq", "dq", "gs", "us", "ds")}
        for d in self.ex:
            for k in cols:
                cols[k].append(q(d[k]) if k.endswith("q") else s(d[k]))
        shared = None
        if self.sh:
            shared = tuple(q(self.sh[k]) if k.endswith("q") else s(self.sh[k]) for k in ("gq", "uq", "dq", "gs", "us", "ds"))
        return moe.ExpertTables(self.H, self.I, 8, cols["gq"], cols["uq"], cols["dq"], cols["gs"], cols["us"], cols["ds"],
                                group=self.group, shared=shared, device=device)


def int8_close(e):
    """Gate of the int8-mode results on small layers, e = errors(...). Integer sums are exact and a typical result is 1e-7
    from the CPU engine's, but the fp32 scale sums and expf differ from the CPU's by ulps, which can move one intermediate
    value across a rounding boundary of its int8 code: one code (1/127 of its group's maximum) on one pick shifts that
    row's outputs by up to ~2e-3 of the output range in a layer this small. More than a few such flips fails."""
    return e[0] < 5e-3 and e[1] < 3e-4


def errors(got, ref):
    """(max-rel, mean-abs, norm-rel), the first two normalised: max|a-b| / max|b| and mean|a-b| / mean|b|."""
    got = np.asarray(got, dtype=np.float64); ref = np.asarray(ref, dtype=np.float64)
    d = np.abs(got - ref)
    return (d.max() / max(np.abs(ref).max(), 1e-30), d.mean() / max(np.abs(ref).mean(), 1e-30),
            np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30))


def random_routing(seed, R, E, topk=8):
    return synth.zipf_routing(seed, 0, R, E, topk, 0.0)
