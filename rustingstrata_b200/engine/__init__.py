from .runner import ModelRunner, StepEntry, StepError
from .scheduler import Scheduler, Request, Scheduled, RequestRejected, SchedulerStuck
from .engine import Engine
