"""CPU oracle for rapid_h3_b200 -- TEST INFRASTRUCTURE ONLY.

A plain PyTorch (CPU, fp32/int) restatement of the quantized-op semantics of the Rapid-H3 node
pack, used as the checker in tests/, in __graft_entry__.smoke() and as the timed CPU baseline of
bench.py. Nothing in the product package imports it, and it never runs on the product path.

Pinning: `linear.py` is checked against golden vectors produced by importing the reference's own
`custom_nodes/rapid_h3/kernels.py` (tests/golden/make_golden.py). The pieces the reference only
implements in CUDA for sm_121 or does not contain at all (fixed-order RMSNorm sums, the block-64 /
fp8-V attention variant, cross-attention, the conv3d decoder) have no reference vectors:
parity unpinned for those; the oracle defines their arithmetic and says so where they are defined.
"""
