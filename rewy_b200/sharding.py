"""(batch, head) sharding of one backward problem across ranks.

Every quantity of the delta-rule backward is per (batch, head) (no cross-head or cross-batch term), so ranks work
on disjoint slices with no collective on the data path.  Batch-major contiguous slices are preferred; when there
are more ranks than batch elements the heads of each batch element are split too.
"""


def shard(B, H, world, rank):
    """Returns (batches, heads): the batch indices and head indices rank `rank` of `world` owns.
    The union over ranks covers every (b, h) exactly once."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("need 0 <= rank < world")
    if world <= B:
        if B % world:
            raise ValueError(f"batch {B} is not divisible by {world} ranks")
        per = B // world
        return list(range(rank * per, (rank + 1) * per)), list(range(H))
    if world % B or H % (world // B):
        raise ValueError(f"cannot split B={B}, H={H} over {world} ranks")
    parts = world // B
    per = H // parts
    return [rank // parts], list(range((rank % parts) * per, (rank % parts + 1) * per))
