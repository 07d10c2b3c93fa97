from .launch_server import main

main()
