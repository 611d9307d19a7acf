"""CPU oracle for the EMA scan: test infrastructure only.

Only tests/, the smoke check and the CPU-baseline / reference arm of bench.py may import this
package.  The product (the CUDA library and its Python host code) never does.
"""
