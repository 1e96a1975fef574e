from .step import ModelRunner, RowInput
