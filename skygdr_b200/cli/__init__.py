"""Command-line programs with the reference's flags and output lines, on this runtime's kernels."""
