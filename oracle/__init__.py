"""CPU oracle for the b200 backend: test infrastructure, never a product code path.

Only tests/, the smoke entry point and bench.py's CPU legs may import this package.
"""
