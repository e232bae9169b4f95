"""CPU oracle of the MoE path (test infrastructure; see oracle/moe_oracle.cpp).

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this package.
"""
