from .decoder import DecoderModel
from . import opt  # noqa: F401  registers OPTForCausalLM; another built-in architecture is one more line here
from . import vononex  # noqa: F401  registers Vononex
from . import pifelix  # noqa: F401  registers Pifelix
from . import tutelix  # noqa: F401  registers Tutelix
from . import vozirax  # noqa: F401  registers Vozirax
