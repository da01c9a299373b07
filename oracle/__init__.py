"""CPU oracle for the quantized-weight matmul path.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, ``__graft_entry__.smoke()`` and
the CPU legs of ``bench.py``; never by the product package.  See ``ref.py`` for
the functions and ``gguf_ref.c`` for the scalar restatement of the reference's
decoder (csrc/ck/gguf_decode.cuh:13-149).
"""
