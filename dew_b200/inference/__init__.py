from .pages import OutOfPages, PageLedger, chain_hash
from .serving import Server, Ticket
from .tasks import TextGeneration, pipeline

__all__ = ["Server", "Ticket", "TextGeneration", "pipeline", "PageLedger", "OutOfPages", "chain_hash"]
