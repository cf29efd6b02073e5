from .random import set_seed
