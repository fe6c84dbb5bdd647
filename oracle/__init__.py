"""TEST INFRASTRUCTURE: CPU oracle of the reference's W8A8 semantics.

Only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` may import this package, and only as
the checker or as the timed CPU baseline.  The product (the ``torch_int``
package and ``libtorch_int_b200.so``) never imports it and has no CPU path.
"""
