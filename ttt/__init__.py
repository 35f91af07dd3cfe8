"""Entry-point aliases: ``python -m ttt.train``, ``python -m ttt.generate`` and ``python -m ttt.data`` run the same
programmes as ``python -m dttt_b200.train | generate | data`` (the module names the reference's users type)."""
