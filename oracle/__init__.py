"""CPU oracle for the INT8 decode-attention / quantiser / fused-MLP path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; it is used by ``tests/``, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` as the checker
and the timed CPU baseline, never as the product path.

Every function restates, in numpy (or, for the timed CPU baseline, in CPU
torch), the algorithm of the reference implementation and cites the
reference file:line it follows.  Parity status: PINNED -- the restatements
are checked in ``tests/test_oracle_golden.py`` against vectors produced by
importing the reference's own Python functions
(``tests/golden/make_golden.py`` is the generating script).
"""
from . import quant, decode, mlp  # noqa: F401
