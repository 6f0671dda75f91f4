"""CPU restatement of the reference's KV-cache / RoPE / chunked-GQA path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package may import this
package: it exists so that tests, the smoke check and the CPU-baseline leg of
the benchmark can compare the CUDA path against an independent NumPy statement
of the reference algorithm (Strata / ``ollm``; the MLX originals cannot run on
a machine without Apple's MLX runtime).

Parity pinning
--------------
* attention: pinned.  ``oracle.attention`` is checked against the outputs of
  the reference's own NumPy oracle ``grouped_attention_reference``
  (tests/test_mlx_attention.py:17-40), generated in a container that holds the
  reference and committed as fixtures under ``tests/golden/`` together with the
  generating script.
* RoPE: pinned the same way against the inline NumPy half-rotation reference of
  tests/test_mlx_generation.py:259-280.
* concat KV cache: pinned against the arange-valued states and the expected
  lengths / error fragments of tests/test_mlx_kvcache.py:22-93.
* decoder glue (RMSNorm / linear / SiLU): pinned against outputs of the
  reference's ``CPUReferenceExecutor`` arithmetic (backends/cpu_reference.py:
  230-369) committed as fixtures.
* parity unpinned: everything the reference does not have -- page tables and
  allocator order, ragged per-sequence lengths, RoPE linear scaling, host
  eviction, KV-head sharding.  Their oracle is *defined* here as the restated
  reference function applied per sequence to the logical K/V that a page table
  denotes (``oracle.paged``).
"""
