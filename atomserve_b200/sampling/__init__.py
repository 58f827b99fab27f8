from atomserve_b200.sampling.sampler import Sampler

__all__ = ["Sampler"]
