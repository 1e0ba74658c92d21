"""Engine core: sequences, block manager, scheduler, model runner, step loop, compression control."""
