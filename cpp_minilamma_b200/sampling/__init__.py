from .sampler import GREEDY_TEMPERATURE, MAX_TOP_K, DeviceSampler, SamplingParams
