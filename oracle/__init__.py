"""CPU restatements of the reference algorithms. Test infrastructure: only tests/, the smoke check and the
benchmark's CPU-baseline leg may import this package."""
