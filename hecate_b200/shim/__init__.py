"""Modules with the names and entry points of the reference's torch extensions for the MoE expert path, forwarding to the C ABI
of libhecate_moe_b200.so, so that the reference's dispatcher (runtime/tier/tier_split.py) runs with only its extension-loading
lines changed:

    from hecate_b200.shim import moe4, moe4p, moe4t, cn       # instead of the four _load_ext(...) calls, tier_split.py:65-81

    moe4.forward / scratch / combine / dequant     runtime/tier/moe4/moe4.cu:916-925
    moe4t.forward / scratch, moe4p.forward / scratch   runtime/tier/moe4/moe4t.cu:526-530, moe4p.cu
    cn.combine_norm                                runtime/tier/cn.cu:190-210

Entry points that exist only to talk to the reference's other processors (moe4.handoff, moe4.stage, cn.combine_norm_pdl's CPU
flags) and the test-only moe4t.gemm raise: there is no second processor behind this path.
"""
