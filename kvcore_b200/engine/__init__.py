"""Engine: step function, model runner, scheduler, engine core and the offline entry point."""
