"""CPU oracle of the SpMM / SDDMM hot path -- test infrastructure only.

Nothing under ``featgraph_b200`` imports this package; only ``tests/``,
``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline / reference arm do.
"""
