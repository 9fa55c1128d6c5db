"""CPU oracle for the Qwen3-0.6B and SigLIP paths.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this directory; only the tests, the smoke check
and the benchmark's CPU-baseline / reference legs do, and only as the checker.

Two layers live here:

* ``qwen3_hf`` / ``siglip_hf`` build the Hugging Face ``transformers`` eager modules that the
  reference itself loads and validates against (reference ``src/ittai/qwen3/model.py:19,32-37``
  and ``src/ittai/siglip/kernel.py:675,701-702``).  ``transformers`` is a third-party dependency
  of the reference (it pins 5.21.0; this image has 5.5.0) and holds the path's arithmetic.
* ``qwen3_ref`` / ``siglip_ref`` restate that arithmetic in plain fp32 tensor operations with every
  bf16 rounding point written out, so each CUDA phase has a line-by-line CPU counterpart.

Parity pin: the reference ships no tests, golden vectors or fixtures, so the restatement is pinned
against outputs of the Hugging Face modules run in this image (``tests/golden/make_golden.py``
writes them, ``tests/test_oracle.py`` checks them).
"""
