"""CPU oracle for the GGUF block decode path -- test infrastructure only.

Nothing in the ``pfhe_b200`` package imports this directory.  Only the test
suite, the smoke check and the CPU-baseline / reference legs of ``bench.py``
use it, and only as the checker or as the timed CPU baseline.

Parity status: pinned.  The vectors under ``tests/golden/`` were produced by
executing the reference's own functions
(``src/phfe/inference/gguf_loader.py:407-554`` followed by the cast at
``:377-378``); ``tests/test_oracle.py`` checks all three restatements here
(``np_oracle``, ``c_oracle``, ``loop_port``) against them bit for bit.
"""
