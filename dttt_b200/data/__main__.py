from .prep import main

main()
