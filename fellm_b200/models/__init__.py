from .model import ARRANGEMENTS, Block, Model, build_model, normed, register_arrangement
