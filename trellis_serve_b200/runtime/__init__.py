"""Run-time pieces above the kernels: the `linear` operator with its row-count dispatch and the decode layer set."""
