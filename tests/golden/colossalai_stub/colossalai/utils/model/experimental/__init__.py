class LazyTensor:
    pass
