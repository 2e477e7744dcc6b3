"""lighthouse_b200: an sm_100a (B200) execution backend for the hot path of llvm/lighthouse —
``linalg.matmul`` with fused epilogues, flash attention, and the nanoGPT / Llama decoder
blocks built from them — behind Lighthouse's own Python surface (``execution.Runner``, the
memory-manager protocol, ``lh-run``, pipeline descriptors).

The arithmetic runs in ``_lib/liblh_b200.so`` (hand-written CUDA, C ABI in
``include/lh_b200.h``); build it with ``python -m lighthouse_b200.build``. There is no CPU
fallback: without the library, or without a GPU, execution raises.
"""

__version__ = "0.1.0"
