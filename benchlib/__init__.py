"""Measurement helpers of bench.py: the seeded synthetic graphs and the sharded-layer benchmark leg."""
