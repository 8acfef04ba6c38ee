"""How work is split over the GPUs of one box (one process per GPU).

The reference has no multi-GPU code; its README rows for 4 GPUs imply
independent windows per GPU.  Two splits exist here:
  * windows: contiguous blocks of global windows per rank, no communication;
  * rows of ONE window: contiguous blocks of rows per rank, one all-reduce of the
    gradient partials per leapfrog step.
"""


def window_block(rank, world, windows):
    """Global windows [w0, w1) of `rank`; blocks differ by at most one window."""
    return rank * windows // world, (rank + 1) * windows // world


def row_block(rank, world, rows):
    """Rows [r0, r1) of `rank` when one window is sharded by rows."""
    return rank * rows // world, (rank + 1) * rows // world
