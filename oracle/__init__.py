"""CPU oracle for the arithmetic of the sm100 kernel bundle.  TEST INFRASTRUCTURE ONLY.

PyTorch fp32 restatements of every kernel family and of the configuration-level models,
dequantising the same E4M3 bytes and fp32 scales the AIM file carries.  Only ``tests/``,
``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline leg import this package; the
product (``aginfer_b200``) never does.

Parity status: UNPINNED by the reference for the arithmetic layer.  wenhuiNi/AgInfer ships
no model kernels, no CPU execution path and no golden vectors for any model op (its only
kernel is ``tests/vector_add.cu``; ``compiler.py:99-105`` declares ``cpu_fallback: False``),
and the model definitions it packages (Qwen2.5-VL, GR00T-N1.5, LingBot-VLA) live in
third-party projects that are not part of its tree.  This oracle therefore *defines* the
arithmetic from the published shapes and the public descriptions of those architectures;
each choice it makes is written where it is made.  The format layer (plan bytes, AIM bytes,
loader answers) is pinned against the reference itself: see ``tests/golden``.
"""
