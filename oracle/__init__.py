"""TEST INFRASTRUCTURE ONLY: CPU restatement of the reference's mixed-precision linear path.

Nothing in ``rdquant_b200`` imports this package.  It is used by ``tests/``, by
``__graft_entry__.smoke()`` and by the ``cpu_baseline`` / ``--impl reference`` legs of
``bench.py`` as the checker and the timed CPU baseline, never as the product path.
"""
