from .model import OPTForGreedySearch, OPTForSampling
