from .model import Block, Model, build_model
