"""CPU restatements of the reference's arithmetic: test infrastructure only.

Nothing under flagtree_b200/ imports this package.  Importers are limited to tests/, the
smoke check in __graft_entry__.py and the CPU-baseline / reference arm of bench.py.
"""
