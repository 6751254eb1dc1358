from .dataloader import SeedGenerator
from .block import Block, create_block_from_coo, create_block_from_csc

__all__ = ["SeedGenerator", "Block", "create_block_from_coo", "create_block_from_csc"]
