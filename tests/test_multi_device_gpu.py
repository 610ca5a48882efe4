"""One process driving two GPUs through the library: everything the host side keeps per device (SM counts, the kernels'
shared-memory attributes, the built-in scratch address of hmoe_decode_noalloc) must be set up on each device, not once per
process. Needs 2 GPUs, else skipped."""
import ctypes as C

import numpy as np
import pytest

from helpers import HostLayer, errors, random_routing
from hecate_b200 import synth

pytestmark = pytest.mark.gpu


def test_decode_router_prefill_on_two_devices_in_one_process():
    import torch
    from hecate_b200 import moe
    from hecate_b200._lib import lib, vp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    H, I, E, R = 6144, 2048, 4, 9            # the full-width kernels: more than 48 KB of dynamic shared memory everywhere
    hl = HostLayer(3, 0, H, I, range(E), 128, True)
    x = synth.activations(5, 0, R, H)
    wt = synth.router_weight(5, 0, 32, H)
    outs = []
    for d in (0, 1):
        dev = torch.device("cuda", d)
        with torch.cuda.device(dev):
            tabs = hl.upload(dev)
            xt = torch.from_numpy(x).to(dev).to(torch.bfloat16)
            wtt = torch.from_numpy(wt).to(dev).to(torch.bfloat16)
            sel = torch.empty(R, 8, dtype=torch.int64, device=dev); rw = torch.empty(R, 8, dtype=torch.float16, device=dev)
            ws = moe.decode_workspace(H, I, dev)
            y = torch.zeros(R, H, device=dev)
            moe.router_decode(tabs, xt, wtt, None, sel, rw, 1.0, y, ws)             # router (+ set-up), gate_up, down
            y2 = torch.zeros(R, H, device=dev)
            moe.router_fused(xt, wtt, None, None, None, sel, rw, 8, 1.0)
            moe.decode(tabs, xt, sel, rw, y2, ws)                                   # the separate set-up kernel
            y3 = torch.zeros(R, H, device=dev)
            st = tabs.struct()
            L = lib(); L.hmoe_decode_noalloc.restype = C.c_int
            rc = L.hmoe_decode_noalloc(C.byref(st), vp(xt), C.c_int(moe._dt(xt)), vp(sel), vp(rw), C.c_int(R), C.c_int(0), C.c_int(E), C.c_int(0),
                                       vp(y3), None, C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
            assert rc == 0, L.hmoe_last_error()
            pws = moe.prefill_workspace(64, 8, E, H, I, dev)
            xp = torch.from_numpy(synth.activations(6, 0, 64, H)).to(dev).to(torch.bfloat16)
            ps, pw = random_routing(7, 64, E)
            out = torch.zeros(64, H, device=dev)
            moe.prefill(tabs, xp, torch.from_numpy(ps).to(dev), torch.from_numpy(pw).to(dev), out, pws)
            torch.cuda.synchronize(dev)
            assert moe.ws_status(ws) == 0 and moe.ws_status(pws) == 0
            outs.append((sel.cpu().numpy(), y.cpu().numpy(), y2.cpu().numpy(), y3.cpu().numpy(), out.cpu().numpy()))
    (s0, a0, b0, c0, p0), (s1, a1, b1, c1, p1) = outs
    assert np.array_equal(s0, s1) and float(np.abs(a0).max()) > 0
    for u, v in ((a0, a1), (b0, b1), (c0, c1), (a0, b0), (a0, c0), (p0, p1)):      # the same work on either device, by either entry point
        assert errors(u, v)[2] < 1e-3
