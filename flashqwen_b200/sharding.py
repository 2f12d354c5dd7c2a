"""KV-head sharding over G GPUs of one node: which heads a rank owns, the element offsets it passes
to the operators, and how all-gathered per-rank outputs go back to full rows.

Heads are independent in every kernel of the path, so rank g of G owns kv heads
[g*8/G, (g+1)*8/G) and their 4x query heads; block tables, positions and the allocator are replicated
and no collective runs inside attention. The single collective is an all-gather of
out_local [rows, (32/G)*128] when a caller needs full rows.
"""
from dataclasses import dataclass

HEAD_DIM = 128
GROUP = 4


@dataclass(frozen=True)
class HeadShard:
    rank: int
    world: int
    n_kv: int = 8

    def __post_init__(self):
        if self.world <= 0 or self.n_kv % self.world or not 0 <= self.rank < self.world:
            raise ValueError(f"{self.n_kv} kv heads do not shard over {self.world} ranks (rank {self.rank})")

    @property
    def n_heads(self):
        return self.n_kv * GROUP

    @property
    def kv_heads_local(self):
        return self.n_kv // self.world

    @property
    def q_heads_local(self):
        return self.kv_heads_local * GROUP

    @property
    def kv_head_begin(self):
        return self.rank * self.kv_heads_local

    @property
    def q_dim(self):
        return self.n_heads * HEAD_DIM

    @property
    def kv_dim(self):
        return self.n_kv * HEAD_DIM

    @property
    def q_elem_off(self):
        """Element offset of the rank's first q head inside a fused qkv row."""
        return self.kv_head_begin * GROUP * HEAD_DIM

    @property
    def k_off(self):
        return self.q_dim + self.kv_head_begin * HEAD_DIM

    @property
    def v_off(self):
        return self.q_dim + self.kv_dim + self.kv_head_begin * HEAD_DIM

    def cache_columns(self):
        """Slice of the last axis of a full [nb, 2, 16, n_kv*128] cache that this rank stores."""
        return slice(self.kv_head_begin * HEAD_DIM, (self.kv_head_begin + self.kv_heads_local) * HEAD_DIM)

    def out_columns(self):
        return slice(self.kv_head_begin * GROUP * HEAD_DIM, (self.kv_head_begin + self.kv_heads_local) * GROUP * HEAD_DIM)


def reassemble(gathered):
    """[G, rows, (H/G)*128] (all_gather_into_tensor order) -> [rows, H*128]."""
    g, rows, cols = gathered.shape
    return gathered.permute(1, 0, 2).reshape(rows, g * cols)
