"""What a layer keeps per request between steps.

The reference has one kind only: keys and values of every token, for every layer alike
(src/minigpt_infer/cache/paged.py:109-123).  Here a mixer states its need as data and
the cache manager groups layers with equal needs.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values in pages.  ``window``: only the last ``window`` positions are ever
    read again (None: all of them), so older pages can be given back early."""

    n_kv_head: int
    head_dim: int
    window: int | None = None
    # Page geometry of the group these layers form.  None: the cache manager's default page
    # size; and for the pool, the manager's default number of pages, or, with a window, as many as
    # every request slot can hold at once (a window's length plus the portion being written never
    # needs more), if that is fewer.
    page_tokens: int | None = None
    num_pages: int | None = None
    # Size of a value head where it differs from a key head's (None: ``head_dim``).
    v_head_dim: int | None = None
    # Queries read only the keys of their own block of this many positions (blocks counted from
    # position 0): the pages of blocks that are over can be given back (None: no such mask).
    block: int | None = None
    # A token's values are the first ``v_head_dim`` features of its key row: no value pages are kept, attention
    # reads the values out of the key pages (a latent that serves as both).
    values_in_keys: bool = False

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim

    def __post_init__(self) -> None:
        if self.n_kv_head <= 0 or self.head_dim <= 0 or self.value_dim <= 0:
            raise ValueError("n_kv_head, head_dim and v_head_dim must be positive")
        if self.window is not None and self.window <= 0:
            raise ValueError("window must be positive when given")
        if self.block is not None and self.block <= 0:
            raise ValueError("block must be positive when given")
        if self.page_tokens is not None and self.page_tokens <= 0:
            raise ValueError("page_tokens must be positive when given")
        if self.num_pages is not None and self.num_pages <= 0:
            raise ValueError("num_pages must be positive when given")
        if self.values_in_keys and self.value_dim > self.head_dim:
            raise ValueError("values that live in the key rows cannot be longer than a key row")


@dataclass(frozen=True)
class FixedStateSpec:
    """A tensor of fixed shape per request, living in a slot of the state pool."""

    shape: tuple[int, ...]
    dtype: str = "float32"


@dataclass(frozen=True)
class PagedKVWithStateSpec:
    """Both at once: keys and values in pages and a tensor of fixed shape in the request's state slot (a layer
    whose mixer runs an attention and a recurrence side by side).  The pages join the group of layers with an equal
    ``pages`` spec; the layer's view of the cache carries its ``state`` beside them."""

    pages: PagedKVSpec
    state: FixedStateSpec
