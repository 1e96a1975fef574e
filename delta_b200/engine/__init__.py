from .engine import LMBackend
from .scheduler import Request, Scheduler
from .step import ModelRunner, RowInput
