"""TEST INFRASTRUCTURE: ctypes loader for the CPU oracle (oracle/oracle.c).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs import this
package.  The product package never does.
"""
from .pyoracle import *  # noqa: F401,F403
