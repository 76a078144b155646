"""Output-row sharding of a dense quantized layer across ranks (one process per GPU).

Rows (output channels) are independent units: rank r owns the contiguous band
[r*N/G, (r+1)*N/G) of W, repacks it locally and computes y_r = W_r x.  The one
exchange step is an all-gather of the y bands; because the bands are contiguous
and equal, the gathered [G][M][N/G] buffer is y for M = 1 and a strided view for
M > 1.  The reference has no multi-GPU path; this layer is new.
"""


def row_band(n_rows, world, rank, align=1):
    """(first_row, rows) of `rank`; bands are equal and `align`-row aligned."""
    if n_rows % (world * align) != 0:
        raise ValueError(f"{n_rows} rows do not split into {world} bands of a multiple of {align}")
    per = n_rows // world
    return rank * per, per


def raw_band_bytes(n_rows, in_dim, world, rank, block_elems, block_bytes):
    """Byte range of a rank's band inside a row-major block-quantized tensor."""
    first, rows = row_band(n_rows, world, rank)
    row_bytes = in_dim // block_elems * block_bytes
    return first * row_bytes, rows * row_bytes


def gathered_to_token_major(gathered, world, batch, rows_per_rank):
    """[G][M][N/G] all-gather result -> [M][N] view (no copy for M = 1)."""
    return gathered.view(world, batch, rows_per_rank).permute(1, 0, 2).reshape(batch, world * rows_per_rank)
