"""CPU checker for the paged-KV path -- TEST INFRASTRUCTURE, not part of the product.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / ``--impl reference`` legs of
``bench.py`` may import this package.  The shipped package never does: its operators run on the
GPU through ``libivab.so`` or raise.
"""
