"""TEST INFRASTRUCTURE ONLY: CPU oracle for the small-batch matmul path.

Only tests/, the smoke check and the CPU-baseline leg of bench.py may import this
package; the product (fastgate_b200) never does.
"""
