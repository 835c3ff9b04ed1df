"""Test infrastructure: the CPU oracle for the predictive-coding train-step path.

``oracle.ref``       – ctypes binding of the reference's own CPU code compiled by
                       ``oracle/build_ref.py`` into ``oracle/_ref/``.
``oracle.pc_oracle`` – a numpy restatement of the same algorithm, pinned against
                       ``oracle.ref`` and against fixtures under ``tests/golden``.

Only tests, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py``
may import this package; the product never does.
"""
