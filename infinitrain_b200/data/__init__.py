from .dataset import (DataLoader, Dataset, DeviceFeeder, DistributedDataLoader, TinyShakespeareDataset, write_token_file)
from .tokenizer import Tokenizer, write_tokenizer_file
