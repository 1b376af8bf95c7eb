"""Data loading (crates/axonml-data)."""
from .collate import Collate, DefaultCollate, StackCollate, concat_tensors, stack_tensors
from .dataloader import Batch, DataLoader, DataLoaderIter, GenericDataLoader, GenericDataLoaderIter
from .dataset import (ConcatDataset, Dataset, InMemoryDataset, MapDataset, SubsetDataset, TensorDataset,
                      random_split)
from .sampler import (BatchIter, BatchSampler, DistributedSampler, RandomSampler, Sampler, SequentialSampler,
                      SubsetRandomSampler, WeightedRandomSampler)
from .transforms import (Clamp, Compose, DropoutTransform, Flatten, Lambda, Normalize, RandomCrop,
                         RandomFlip, RandomNoise, Reshape, Scale, ToTensor, Transform)
