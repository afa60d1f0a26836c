"""CPU checkers for the matmul path (test infrastructure, never shipped).

Only tests/, ``__graft_entry__.smoke()`` and the CPU legs of ``bench.py`` may
import this package.
"""
