"""TEST INFRASTRUCTURE: CPU restatement of the reference's quantized path.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may
import this package.  ``oracle.c`` wraps the C restatement
(oracle/qpath_oracle.c, built by ``make -C oracle``); ``oracle.np_ref`` is an
independent numpy statement of the same formulas used to cross-check the C.
"""
