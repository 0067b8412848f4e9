"""TEST INFRASTRUCTURE — the parity oracle.  Not part of the product.

CPU restatement of the reference's per-chunk optimizer step, used only as the
checker: by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline
leg of ``bench.py``.  Nothing under ``patrickstar_b200/`` imports this package.

Parity status: PINNED — ``adam_oracle.c`` is checked bit-for-bit against the
reference's own AVX build (``oracle/_ref``, compiled from the reference
checkout by ``oracle/build.py``) and against golden vectors generated from that
build and from the reference's Python ``DynamicLossScaler``
(``tests/golden/``).

Modules
  adam_oracle.c     C restatement of cpu_adam.cpp / cpu_adam.h (+ casts, inf/nan test)
  port.py           ctypes binding of the C restatement
  ref.py            loader of the compiled reference module (oracle/_ref)
  scaler_oracle.py  Python restatement of loss_scaler.py and of the engine's config mapping
  step_oracle.py    FP16Adam.step protocol (skip / step count / scale update) over the C oracle
  build.py          build recipe
"""
