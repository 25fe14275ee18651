from .runner import ModelRunner, StepEntry, StepError
from .scheduler import Scheduler, Request, Scheduled, RequestRejected
from .engine import Engine
