"""CPU oracle for the quantized-linear + KV-cache-attention path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import this
directory; the only legitimate callers are the test-suite, the smoke check
and the CPU-baseline / reference arms of the benchmark driver.

Every function restates, in plain torch-CPU / numpy arithmetic, what the
reference computes for one operator, and cites the reference file:line it
follows (paths are relative to the reference project root).

Pinning status
--------------
* int8 / fp8 activation quantizers, the per-token x per-channel dequant
  formula, AWQ unpack / dequantize, RMSNorm, RoPE and the KV-cache update are
  pinned against outputs of the reference's own importable pure-torch code
  (fixtures under tests/golden, produced by tests/golden/make_golden.py).
* The AWQ fused dequant-GEMM is pinned against the reference's Triton kernel
  executed by the Triton CPU interpreter (small shapes, same fixtures).
* The int8 / fp8 GEMM epilogues are pinned against the procedures of the
  reference's three unit tests (runtime/unittest/test_*.py): same shapes,
  same construction, same tolerances.
* Attention: the reference delegates the arithmetic to the un-vendored pip
  package flash-attn (only pin: the comment "2.4.2 -> 2.7.4" at
  runtime/nn_models/modules/nonlinear/attn.py:11) and ships no test or
  vector for it; the oracle restates the published operator semantics and is
  pinned on the GPU against the installed flash_attn package called with the
  reference's keyword sets (tests/test_gpu_attention_pin.py).  On a machine
  without that package those tests skip and attention parity is unpinned.
"""
