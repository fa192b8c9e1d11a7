"""TEST INFRASTRUCTURE, NOT PRODUCT.

CPU restatements of the reference's routed-expert MoE path (bertholomus/TensorFold), used as the checker by
``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs, and by nothing else: no module under
``tensorfold_b200/`` imports, links or executes anything here.

* ``cpu_moe.c`` / ``cpu.py`` - plain C (OpenMP) restatement of routing, plan, the affine-row kernel and the whole
  affine layer; also the timed CPU baseline.
* ``affine.py``  - numpy restatement of the MLX affine 4-bit group-64 format and float64 layer references.
* ``exl3.py``    - numpy restatement of the EXL3 trellis format, codebooks, Hadamard rotations and layer.
* ``build.py``   - compiles ``cpu_moe.c``;  ``build_ref.py`` compiles the reference's own Metal header as C++ into
  ``oracle/_ref/`` where the reference tree is mounted (this container only).
"""
