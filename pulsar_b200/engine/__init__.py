from .loading import load_model, torch_dtype
from .runner import ModelRunner, StepEntry, StepError
