"""Same module layout as the reference's `kernels/` package."""
