"""TEST INFRASTRUCTURE ONLY - CPU restatement of the reference's naive executor.

Nothing in the shipped package imports this directory.  It is used by ``tests/``, by
``__graft_entry__.smoke()`` as the checker and by ``bench.py`` for the CPU baseline leg.
Parity status: PINNED - `tests/test_oracle_golden.py` checks it against input/output
vectors produced by running the reference's own naive torch path
(``tests/golden/make_golden.py`` is the script that generated them).
"""
