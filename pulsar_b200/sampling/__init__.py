from .sampler import GenerationParams, Sampler, make_generator
