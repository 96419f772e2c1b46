from .step import BufferPool, Runner, StepContext, StepEntry, StepError
