"""CPU oracle for the backward + gradient-synchronisation path.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by
the CPU leg of ``bench.py``; never by the product package ``singa_b200``.

``oracle.cpu``   ctypes front end of ``oracle.c`` (plain C, OpenMP).
``oracle.comm``  numpy restatement of the communicator arithmetic
                 (bucket policy, fp16 sync, threshold / top-K sparsification).
``oracle.build`` gcc recipe for ``liboracle.so`` and for the objects compiled
                 straight from the reference tree into ``oracle/_ref/``.
"""
