from .allocators import PageAllocator, SlotAllocator
from .sequence_cache import (PAGE_SIZE, KVRequirement, KVView, SequenceCache, StateRequirement, StateView)
