from .module import ElixirModule
from .optimizer import ElixirOptimizer, OptimState
from .plan import ChunkPlan, SearchResult, simple_plan, simple_search

__all__ = ['ChunkPlan', 'ElixirModule', 'ElixirOptimizer', 'OptimState', 'SearchResult', 'simple_plan', 'simple_search']
